"""``prism-serve`` console entry (reference ``prism_infer/serving/cli.py:43-93``).

    prism-serve --model <dir | random:tiny> [--engine-config file.json] [--host H] [--port P]
                [--ingress-capacity N] [--max-restarts 0] [--restart-window 0] [--log-level info]

``--engine-config`` is a JSON object of ``LLM`` keyword options; a single uvicorn worker is
used because one process owns the GPUs.
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

PROTECTED = {"model", "metrics_sink", "clock_ns", "request_id_allocator", "runner_group", "weights"}


def load_engine_options(path: str | None) -> dict[str, object]:
    if path is None:
        return {}
    try:
        payload = json.loads(Path(path).read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as exc:
        raise ValueError(f"cannot read engine config {path}: {exc}") from exc
    if not isinstance(payload, dict) or any(not isinstance(k, str) for k in payload):
        raise ValueError("engine config must be a JSON object with string keys")
    clash = sorted(PROTECTED & payload.keys())
    if clash:
        raise ValueError(f"engine config cannot override CLI-owned fields: {clash}")
    return payload


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="prism-serve", description="Serve Qwen3-VL over HTTP / SSE")
    ap.add_argument("--model", required=True)
    ap.add_argument("--engine-config", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--ingress-capacity", type=int, default=64)
    ap.add_argument("--max-restarts", type=int, default=0,
                    help="after a failed engine step rebuild the engine and run the open greedy requests again, this many times (0: a failure is final)")
    ap.add_argument("--restart-window", type=float, default=0.0,
                    help="seconds; only restarts within this window count against --max-restarts (0: all of them do)")
    ap.add_argument("--log-level", default="info")
    return ap


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    options = load_engine_options(args.engine_config)
    import uvicorn

    from ..llm import LLM
    from .app import create_app
    from .runtime import ServingRuntime

    runtime = ServingRuntime(lambda: LLM(args.model, **options), ingress_capacity=args.ingress_capacity,
                             max_restarts=args.max_restarts, restart_window_s=args.restart_window)
    uvicorn.run(create_app(runtime, model_name=os.path.basename(os.path.normpath(args.model)) or args.model), host=args.host, port=args.port, log_level=args.log_level, workers=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
