"""Answer quality of the dense and the compacted multimodal prefix on repeated visual context
(reference ``benchmarks/bench_working_set_quality.py``).

Input is a JSONL of materialised quality records (``analysis/quality_materialization.py``): each
has ``sample_id``, ``question``, ``media`` (content-addressed files under ``--media-root``) and
either ``options`` + ``answer`` (a letter; multiple choice) or ``answers`` (free text, scored
with ANLS >= 0.5), or - MVBench video records as ``utils/materialize_mvbench_media`` completes them -
``candidates`` + ``answer_index`` with one ``video`` / ``frames`` media entry and an optional time window:
``--video-frames`` frames are sampled at segment centres (inside the window when there is one), the prompt is
the benchmark's ``Question / Option / (A) ...`` form and the answer letter is parsed the benchmark's way.  Records are grouped by identical ordered media; only groups with at least
two questions are kept, and every prompt puts the media first so that all questions of a group
share one visual prefix.  Inside a group the first question runs cold and stores the prefix,
the others reuse it - which is exactly the situation in which the compacted prefix could cost
accuracy, because every later question sees only the visual tokens kept for the first.

Each stage (``dense_prefix``: scaled-FP8 KV; ``compact_prefix``: scaled-FP8 KV + physical visual
compaction) runs on its own engine and appends one line per sample to ``<out>/<stage>.samples.jsonl``
(rewritten atomically after every group).  ``--resume`` keeps the complete groups already there
and continues; lines that do not match the plan are refused.  ``<out>/summary.json`` holds each
stage's accuracy, the prefix reuse observed and the paired comparison on the samples whose
visual tokens the compact stage actually deleted.

    python benchmarks/bench_working_set_quality.py --records muirbench.jsonl --media-root data/quality --out runs/quality
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from prism_infer_b200.analysis import quality_metrics as qm  # noqa: E402
from prism_infer_b200.analysis import working_set_quality as wsq  # noqa: E402
from prism_infer_b200.analysis.identity import canonical_json_sha256  # noqa: E402
from prism_infer_b200.analysis.quality_materialization import (safe_materialized_path, sha256_file, verify_materialized_records,  # noqa: E402
                                                               write_json_atomic, write_jsonl_atomic)

STAGES: dict[str, dict[str, Any]] = {
    "dense_prefix": dict(compression_mode="scaled_fp8_kv"),
    "compact_prefix": dict(compression_mode="visual_compact_scaled_fp8", visual_pruning_keep_ratio=0.6, visual_pruning_min_keep_tokens=768),
}
MARKER = "<image>"
CHOICE_HINT = "Answer with the option's letter from the given choices directly."


def load_records(path: str | Path) -> list[dict[str, Any]]:
    rows = [json.loads(line) for line in Path(path).read_text(encoding="utf-8").splitlines() if line.strip()]
    ids = [r.get("sample_id") for r in rows]
    if len(set(map(str, ids))) != len(ids):
        raise ValueError("duplicate sample_id in the records")
    for r in rows:
        has_choice = isinstance(r.get("options"), list) and isinstance(r.get("answer"), str)
        has_text = isinstance(r.get("answers"), list) and bool(r["answers"])
        if not isinstance(r.get("question"), str) or int(has_choice) + int(has_text) + int(is_video_record(r)) != 1:
            raise ValueError(f"record {r.get('sample_id')!r} needs a question and one of options+answer, answers, "
                             "or candidates+answer_index with a video / frames source")
    return rows


def is_video_record(record: Mapping[str, Any]) -> bool:
    """An MVBench question: candidates with the index of the right one, and a single video or frame-directory source."""
    media = record.get("media")
    idx = record.get("answer_index")
    return (isinstance(record.get("candidates"), list) and isinstance(idx, int) and not isinstance(idx, bool)
            and 0 <= idx < len(record["candidates"]) and isinstance(media, list) and len(media) == 1
            and isinstance(media[0], Mapping) and media[0].get("media_type") in ("video", "frames"))


def evaluable(records: Sequence[Mapping[str, Any]]) -> list[Mapping[str, Any]]:
    """Video records whose media were excluded (absent from the archive, separately licensed) leave the run."""
    return [r for r in records if not is_video_record(r) or r["media"][0].get("materialization_status") == "complete"]


def prompt_for(record: Mapping[str, Any]) -> str:
    if is_video_record(record):
        return qm.mvbench_prompt(record["question"], record["candidates"])
    n = len(record["media"])
    if "options" in record:
        opts = [f"({chr(65 + i)}) {o}" for i, o in enumerate(record["options"])]
        return wsq.build_media_first_prompt(record["question"], n, marker=MARKER, options=opts, hint=CHOICE_HINT)
    return wsq.build_media_first_prompt(record["question"], n, marker=MARKER, hint="Answer the question using a single word or phrase.")


def score(record: Mapping[str, Any], text: str) -> dict[str, Any]:
    if is_video_record(record):
        t = qm.mvbench_score(dict(record), text)
        return {"parsed": t["prediction"], "correct": bool(t["score"]), "score": float(t["score"]), "parse_method": t["parse_method"]}
    if "options" in record:
        picked = qm.parse_choice(text, len(record["options"]))
        return {"parsed": picked, "correct": picked == record["answer"], "score": float(picked == record["answer"])}
    s = qm.anls(text, record["answers"])
    return {"parsed": text.strip(), "correct": s > 0.0, "score": s}


def _load_images(record: Mapping[str, Any], root: str | Path) -> list[Any]:
    from PIL import Image

    out = []
    for m in record["media"]:
        with Image.open(safe_materialized_path(root, m["materialized_path"])) as im:
            out.append(im.convert("RGB").copy())
    return out


def _load_frames(record: Mapping[str, Any], root: str | Path, frames: int, frame_dir_fps: float) -> tuple[list[Any], dict[str, Any]]:
    """The sampled RGB frames of a video record and how they were obtained."""
    from prism_infer_b200.analysis import video_sampling as vs

    m = record["media"][0]
    if m["media_type"] == "frames":
        return vs.sample_frame_manifest(m["frames"], materialized_root=root, frames=frames, fps=frame_dir_fps,
                                        temporal_bound=record.get("temporal_bound"))
    return vs.sample_video_file(safe_materialized_path(root, m["materialized_path"]), frames=frames, temporal_bound=record.get("temporal_bound"))


def verify_media(records: Sequence[Mapping[str, Any]], root: str | Path) -> dict[str, int]:
    """Re-hash every file the run will read: image files, video files and every frame of a frame directory."""
    flat = []
    for r in records:
        for m in r["media"]:
            parts = m["frames"] if m.get("media_type") == "frames" else [m]
            flat.append({"sample_id": r["sample_id"], "media": [{"sha256": p["sha256"], "materialized_path": p["materialized_path"]} for p in parts]})
    return verify_materialized_records(flat, root)


def _resume_lines(path: Path, plan: Sequence[wsq.GroupedQualitySample], resume: bool) -> list[dict[str, Any]]:
    """Lines of complete groups that match the plan's order; a trailing partial group is dropped."""
    if not path.exists():
        return []
    if not resume:
        raise FileExistsError(f"{path} exists: pass --resume to continue it or remove it")
    rows = [json.loads(line) for line in path.read_text(encoding="utf-8").splitlines() if line.strip()]
    for row, item in zip(rows, plan):
        if str(row.get("sample_id")) != str(item.record["sample_id"]) or row.get("media_group_id") != item.media_group_id:
            raise ValueError(f"{path}: line for sample {row.get('sample_id')!r} does not match the plan")
    if len(rows) > len(plan):
        raise ValueError(f"{path} holds more samples than the plan")
    keep = len(rows)
    while keep and keep < len(plan) and plan[keep].question_index != 0:
        keep -= 1  # cut back to a group boundary
    return rows[:keep]


def run_stage(stage: str, plan: Sequence[wsq.GroupedQualitySample], make_engine: Callable[[dict[str, Any]], Any], media_root: str | Path,
              out_dir: Path, *, max_tokens: int, resume: bool, log: Callable[[str], None] = print, video_frames: int = 16,
              frame_dir_fps: float = 3.0) -> list[dict[str, Any]]:
    from prism_infer_b200 import SamplingParams

    path = out_dir / f"{stage}.samples.jsonl"
    rows = _resume_lines(path, plan, resume)
    if len(rows) == len(plan):
        return rows
    llm = make_engine(STAGES[stage])
    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens)
    try:
        i = len(rows)
        while i < len(plan):
            group = [it for it in plan[i:i + plan[i].group_size] if it.media_group_id == plan[i].media_group_id]
            video = is_video_record(group[0].record)
            sampling = None
            if video:
                images, sampling = _load_frames(group[0].record, media_root, video_frames, frame_dir_fps)
            else:
                images = _load_images(group[0].record, media_root)
            deleted = 0
            for it in group:
                before = llm.multimodal_prefix_cache_metadata()
                n_req = len(llm.metrics_snapshot()["engine"]["requests"])
                if video:
                    out = llm.generate_video(prompt_for(it.record), images, sp, use_tqdm=False)
                else:
                    out = llm.generate_interleaved_images(prompt_for(it.record), images, sp, image_marker=MARKER, use_tqdm=False)
                after = llm.multimodal_prefix_cache_metadata()
                metric = llm.metrics_snapshot()["engine"]["requests"][n_req]
                if it.question_index == 0:  # the cold request stored the prefix: what did compaction drop?
                    deleted = int((after["logical_tokens"] - before["logical_tokens"]) - (after["resident_tokens"] - before["resident_tokens"]))
                rows.append({"sample_id": it.record["sample_id"], "media_group_id": it.media_group_id, "question_index": it.question_index,
                             "stage": stage, "prediction": out["text"], **score(it.record, out["text"]),
                             "prefix_hit": after["hits"] - before["hits"] == 1, "cached_tokens": metric["cached_tokens"],
                             "prompt_tokens": metric["prompt_tokens"], "deleted_visual_tokens": deleted})
                if sampling is not None:
                    rows[-1]["sampled_indices"] = sampling["sampled_indices"]
                    rows[-1]["sampled_rgb_identity_sha256"] = sampling["sampled_rgb_identity_sha256"]
            i += len(group)
            write_jsonl_atomic(path, rows)
            log(f"{stage}: {i}/{len(plan)} samples")
    finally:
        llm.exit()
    return rows


def summarize(stage_rows: Mapping[str, Sequence[Mapping[str, Any]]], plan: Sequence[wsq.GroupedQualitySample]) -> dict[str, Any]:
    out: dict[str, Any] = {"record_type": "working_set_quality_summary", "samples": len(plan),
                           "groups": len({it.media_group_id for it in plan}),
                           "plan_sha256": canonical_json_sha256([[str(it.record["sample_id"]), it.media_group_id] for it in plan]), "stages": {}}
    for stage, rows in stage_rows.items():
        later = [r for r in rows if r["question_index"] > 0]
        out["stages"][stage] = {**wsq.summarize_stage_samples(rows), "mean_score": sum(r["score"] for r in rows) / len(rows) if rows else 0.0,
                                "repeat_questions": len(later), "repeat_prefix_hits": sum(1 for r in later if r["prefix_hit"]),
                                "cached_tokens": sum(r["cached_tokens"] for r in rows), "prompt_tokens": sum(r["prompt_tokens"] for r in rows)}
    if {"dense_prefix", "compact_prefix"} <= set(stage_rows):
        out["paired_deleted_subset"] = wsq.paired_deleted_subset(stage_rows["dense_prefix"], stage_rows["compact_prefix"])
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--records", required=True)
    ap.add_argument("--media-root", required=True)
    ap.add_argument("--out", required=True, help="output directory")
    ap.add_argument("--model", default=os.environ.get("PRISM_MODEL_PATH", "random:qwen3-vl-8b"))
    ap.add_argument("--stages", default="dense_prefix,compact_prefix")
    ap.add_argument("--max-groups", type=int, default=None)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--pages", type=int, default=1024)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--device", default=None)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--video-frames", type=int, default=16, help="frames sampled from a video record")
    ap.add_argument("--frame-dir-fps", type=float, default=3.0, help="frame rate at which frame directories were exported")
    args = ap.parse_args(argv)
    stages = [s for s in args.stages.split(",") if s]
    for s in stages:
        if s not in STAGES:
            ap.error(f"unknown stage {s!r}; known: {sorted(STAGES)}")
    records = evaluable(load_records(args.records))
    media_check = verify_media(records, args.media_root)
    sampling_identity = {"video_frames": args.video_frames, "frame_dir_fps": args.frame_dir_fps} if any(map(is_video_record, records)) else None
    plan = wsq.select_multi_question_groups(records, max_groups=args.max_groups, sampling_identity=sampling_identity)
    if not plan:
        raise SystemExit("no media group has two or more questions")
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    def make_engine(extra: dict[str, Any]):
        from prism_infer_b200 import LLM

        return LLM(args.model, device=args.device, tensor_parallel_size=args.tp, max_model_len=8192, max_num_batched_tokens=8192,
                   max_num_seqs=2, max_chunk_size=8192, kvcache_block_size=256, num_kvcache_blocks=args.pages, cpu_kv_cache_ratio=0.0,
                   enable_prefix_caching=True, **extra)

    rows = {s: run_stage(s, plan, make_engine, args.media_root, out_dir, max_tokens=args.max_tokens, resume=args.resume,
                         video_frames=args.video_frames, frame_dir_fps=args.frame_dir_fps) for s in stages}
    summary = summarize(rows, plan)
    summary["config"] = {"model": args.model, "stages": stages, "max_tokens": args.max_tokens, "pages": args.pages, "tp": args.tp,
                         "video_frames": args.video_frames, "frame_dir_fps": args.frame_dir_fps, "stage_options": {s: STAGES[s] for s in stages}}
    # what went in: the record file by content, the media that were re-hashed, the source tree and the GPU
    import harness

    summary["inputs"] = {"records_file_sha256": sha256_file(args.records), "evaluated_records_sha256": canonical_json_sha256(list(records)),
                         "media_verified": media_check}
    summary["provenance"] = harness.provenance()
    write_json_atomic(out_dir / "summary.json", summary)
    print(json.dumps({k: summary[k] for k in ("samples", "groups", "stages") if k in summary} | {"paired": summary.get("paired_deleted_subset")}))


if __name__ == "__main__":
    main()
