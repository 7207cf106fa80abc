"""Measure the dense prefix pages of every media group, then build the shared working-set plan
(reference ``benchmarks/build_working_set_plan.py``).

The working-set regimes (fit / knee / pressure) are defined by how many KV pages the groups'
multimodal prefixes occupy when stored densely, so that number is measured, not estimated: one
cold, media-first request per group on an engine with the dense prefix cache, and the growth
of the cache's resident pages is the group's ``dense_prefix_pages``.  Every finished measurement
is written to the page artifact atomically (temporary file + rename), so an interrupted run
continues with ``--resume`` from the groups already measured; a page artifact made under a
different measurement contract (model, page size, image size, seed, group count) is refused.

    python benchmarks/build_working_set_plan.py --out plan.json [--regime knee] [--pages 220] [--resume]
    python benchmarks/bench_online.py --plan plan.json --variant compact_prefix

With ``--records muirbench.jsonl --media-root data/quality`` the groups are the multi-question media groups of
materialised image records (real images read from the content-addressed tree, every file re-hashed) instead of
synthetic ones; the plan then names each media file and ``bench_online.py --plan ... --media-root ...`` replays it.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from pathlib import Path
from typing import Any, Callable, Sequence

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200.analysis import working_set_plan as wsp  # noqa: E402
from prism_infer_b200.analysis.identity import canonical_json_sha256  # noqa: E402
from prism_infer_b200.analysis.quality_materialization import write_json_atomic  # noqa: E402

PAGE_ARTIFACT_VERSION = 1
PLAN_DOCUMENT_VERSION = 1


def image_for(digest: str, size: int) -> np.ndarray:
    """The synthetic image a media digest stands for (same rule as ``bench_online.py``)."""
    seed = int.from_bytes(hashlib.sha256(digest.encode()).digest()[:8], "little")
    return np.random.default_rng(seed).integers(0, 256, (size, size, 3), dtype=np.uint8)


def file_image_loader(media_root: str | Path, media_paths: dict[str, str]) -> Callable[[str], np.ndarray]:
    """digest -> RGB pixels of the materialised file, its bytes checked against the digest."""
    from PIL import Image

    from prism_infer_b200.analysis.quality_materialization import safe_materialized_path, sha256_file

    def load(digest: str) -> np.ndarray:
        path = safe_materialized_path(media_root, media_paths[digest])
        if sha256_file(path) != digest:
            raise OSError(f"content hash mismatch: {path}")
        with Image.open(path) as im:
            return np.asarray(im.convert("RGB"))

    return load


def measurement_contract(*, model: str, page_tokens: int, image_size: int, seed: int, groups: Sequence[wsp.MediaGroup],
                         records_sha256: str | None = None) -> dict[str, Any]:
    out = {"model": model, "page_tokens": page_tokens, "image_size": image_size, "seed": seed, "kv_mode": "scaled_fp8_kv",
           "prompt": "media_first", "group_ids_sha256": canonical_json_sha256([g.group_id for g in groups])}
    if records_sha256 is not None:  # real media: the pixels come from files, not from (seed, image size)
        out.update(media="materialized_records", records_sha256=records_sha256, image_size=0)
    return out


def load_page_artifact(path: Path, contract: dict[str, Any], *, resume: bool) -> dict[str, Any]:
    if not path.exists():
        return {"artifact_version": PAGE_ARTIFACT_VERSION, "contract": contract, "groups": {}}
    if not resume:
        raise FileExistsError(f"{path} exists: pass --resume to continue it or remove it")
    art = json.loads(path.read_text(encoding="utf-8"))
    if art.get("artifact_version") != PAGE_ARTIFACT_VERSION or art.get("contract") != contract:
        raise ValueError(f"{path} was measured under a different contract")
    for gid, m in art["groups"].items():
        if not isinstance(m.get("dense_prefix_pages"), int) or m["dense_prefix_pages"] <= 0:
            raise ValueError(f"{path}: malformed measurement for group {gid}")
    return art


def measure_group(llm, group: wsp.MediaGroup, image_size: int | Callable[[str], np.ndarray], sp) -> dict[str, int]:
    """One cold media-first request -> growth of the prefix cache.  ``image_size``: the edge of the synthetic
    images, or a loader ``digest -> pixels`` for real media."""
    before = llm.multimodal_prefix_cache_metadata()
    prompt = wsp.media_first_prompt(group.num_images, group.questions[0])
    load = image_size if callable(image_size) else (lambda d: image_for(d, image_size))
    llm.generate_interleaved_images(prompt, [load(d) for d in group.media_digests], sp,
                                    image_marker=wsp.IMAGE_MARKER, use_tqdm=False)
    after = llm.multimodal_prefix_cache_metadata()
    if after["stores"] - before["stores"] != 1 or after["hits"] != before["hits"]:
        raise RuntimeError(f"group {group.group_id[:12]}: the request was not one cold store "
                           f"(stores +{after['stores'] - before['stores']}, hits +{after['hits'] - before['hits']})")
    if after["evictions"] != before["evictions"]:
        raise RuntimeError("the measuring engine evicted a prefix: give it more pages")
    return {"dense_prefix_pages": int(after["resident_pages"] - before["resident_pages"]),
            "prefix_tokens": int(after["logical_tokens"] - before["logical_tokens"]), "images": group.num_images}


def measure_all(groups: Sequence[wsp.MediaGroup], artifact_path: Path, contract: dict[str, Any], make_engine: Callable[[], Any],
                image_size: int | Callable[[str], np.ndarray], *, resume: bool, log: Callable[[str], None] = print) -> dict[str, Any]:
    from prism_infer_b200 import SamplingParams

    art = load_page_artifact(artifact_path, contract, resume=resume)
    todo = [g for g in groups if g.group_id not in art["groups"]]
    if todo:
        llm = make_engine()
        try:
            sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
            for g in todo:
                art["groups"][g.group_id] = measure_group(llm, g, image_size, sp)
                write_json_atomic(artifact_path, art)
                log(f"measured {len(art['groups'])}/{len(groups)}: {g.group_id[:12]} -> {art['groups'][g.group_id]['dense_prefix_pages']} pages")
        finally:
            llm.exit()
    return art


def plan_document(plan: wsp.WorkingSetPlan, contract: dict[str, Any], regime: str, media_paths: dict[str, str] | None = None) -> dict[str, Any]:
    doc = {"plan_version": PLAN_DOCUMENT_VERSION, "regime": regime, "contract": contract,
           "media_groups": [{"group_id": g.group_id, "media_digests": list(g.media_digests), "questions": list(g.questions),
                       "dense_prefix_pages": g.dense_prefix_pages} for g in plan.groups],
           **plan.to_record()}
    if media_paths is not None:
        used = {d for g in plan.groups for d in g.media_digests}
        doc["media_paths"] = {d: p for d, p in sorted(media_paths.items()) if d in used}
    doc["plan_sha256"] = canonical_json_sha256(doc)
    return doc


def load_plan_document(path: str | Path) -> tuple[wsp.WorkingSetPlan, dict[str, Any]]:
    doc = json.loads(Path(path).read_text(encoding="utf-8"))
    body = {k: v for k, v in doc.items() if k != "plan_sha256"}
    if doc.get("plan_version") != PLAN_DOCUMENT_VERSION or canonical_json_sha256(body) != doc.get("plan_sha256"):
        raise ValueError(f"{path}: not a plan document, or edited after it was written")
    groups = [wsp.MediaGroup(g["group_id"], tuple(g["media_digests"]), tuple(g["questions"]), int(g["dense_prefix_pages"]))
              for g in doc["media_groups"]]
    mk = lambda rows: [wsp.PlannedRequest(**r) for r in rows]  # noqa: E731
    plan = wsp.WorkingSetPlan(groups, mk(doc["population"]), mk(doc["measured"]), doc["seed"], doc["alpha"], doc["rate_per_s"],
                              doc["page_budget"], doc["working_set_pages"])
    return plan, doc


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True, help="plan document; the page artifact is written beside it as <out>.pages.json")
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--regime", choices=("fit", "knee", "pressure", "all"), default="knee")
    ap.add_argument("--pages", type=int, default=220, help="KV page budget the regimes are defined against")
    ap.add_argument("--groups", type=int, default=42)
    ap.add_argument("--questions", type=int, default=85)
    ap.add_argument("--min-images", type=int, default=1)
    ap.add_argument("--max-images", type=int, default=8)
    ap.add_argument("--image-size", type=int, default=448)
    ap.add_argument("--requests", type=int, default=600)
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--alpha", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=wsp.DEFAULT_SEED)
    ap.add_argument("--page-tokens", type=int, default=256)
    ap.add_argument("--device", default=None)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--records", default="", help="JSONL of materialised image records: real media groups instead of synthetic ones")
    ap.add_argument("--media-root", default="", help="root of the content-addressed media tree of --records")
    ap.add_argument("--max-groups", type=int, default=None, help="with --records: keep the first N groups in group-id order")
    args = ap.parse_args()
    out = Path(args.out)
    if out.exists():
        raise FileExistsError(f"refusing to overwrite {out}")
    media_paths = None
    loader: int | Callable[[str], np.ndarray] = args.image_size
    if args.records:
        if not args.media_root:
            ap.error("--records needs --media-root")
        records = [json.loads(line) for line in Path(args.records).read_text(encoding="utf-8").splitlines() if line.strip()]
        groups, media_paths = wsp.groups_from_records(records)
        if args.max_groups is not None:
            groups = groups[:args.max_groups]
        if not groups:
            raise SystemExit("no media group of the records has two or more questions")
        loader = file_image_loader(args.media_root, media_paths)
        contract = measurement_contract(model=args.model, page_tokens=args.page_tokens, image_size=0, seed=args.seed, groups=groups,
                                        records_sha256=canonical_json_sha256(records))
    else:
        groups = wsp.synthetic_groups(args.groups, args.questions, seed=args.seed, min_images=args.min_images, max_images=args.max_images,
                                      tokens_per_image=(args.image_size // 32) ** 2 + 2, page=args.page_tokens)
        contract = measurement_contract(model=args.model, page_tokens=args.page_tokens, image_size=args.image_size, seed=args.seed,
                                        groups=groups)

    def make_engine():
        from prism_infer_b200 import LLM

        # analytic upper bound + room for the running request (real media: eight pages per image covers 1024 x 1024 pixels)
        estimate = sum(g.dense_prefix_pages or 8 * g.num_images for g in groups)
        return LLM(args.model, device=args.device, max_model_len=8192, max_num_batched_tokens=8192, max_num_seqs=2, max_chunk_size=8192,
                   kvcache_block_size=args.page_tokens, num_kvcache_blocks=estimate + 64, cpu_kv_cache_ratio=0.0,
                   enable_prefix_caching=True, compression_mode="scaled_fp8_kv")

    art = measure_all(groups, Path(str(out) + ".pages.json"), contract, make_engine, loader, resume=args.resume)
    measured = [wsp.MediaGroup(g.group_id, g.media_digests, g.questions, art["groups"][g.group_id]["dense_prefix_pages"]) for g in groups]
    chosen = wsp.select_groups(measured, args.pages, args.regime)
    plan = wsp.build_plan(chosen, num_requests=args.requests, alpha=args.alpha, rate=args.rate, seed=args.seed, page_budget=args.pages)
    doc = plan_document(plan, contract, args.regime, media_paths)
    write_json_atomic(out, doc)
    print(json.dumps({"out": str(out), "regime": args.regime, "groups": len(chosen), "working_set_pages": plan.working_set_pages,
                      "page_budget": args.pages, "plan_sha256": doc["plan_sha256"]}))


if __name__ == "__main__":
    main()
