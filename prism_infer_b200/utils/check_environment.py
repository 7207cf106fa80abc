"""``python -m prism_infer_b200.utils.check_environment``: print the capability report and
exit non-zero when a requirement is unmet (the reference ships ``scripts/check_environment.py``)."""

from __future__ import annotations

import json
import sys

from ..runtime_capabilities import probe_runtime_capabilities


def main() -> int:
    rep = probe_runtime_capabilities(require_cuda="--allow-cpu" not in sys.argv)
    print(json.dumps(rep.__dict__, indent=1, default=str))
    return 0 if rep.ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
