"""The persistent decode kernel (all decoder layers of a decode step in one launch) against the
per-layer kernel chain it replaces, on the same weights, the same KV pages and the same inputs:
hidden states after the final norm, and the K / V rows written for the new tokens."""

import pytest
import torch

from prism_infer_b200 import ops
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.models.qwen3_vl import AttnMeta, Qwen3VLModel
from prism_infer_b200.models.weights import iter_random_weights
from prism_infer_b200.ops import decode_layers as dl
from prism_infer_b200.ops import native

pytestmark = pytest.mark.gpu


def _model(arch):
    model = Qwen3VLModel(arch, device="cuda", dtype=torch.bfloat16, load_vision=False)
    model.load(iter_random_weights(arch, dtype=torch.bfloat16, device="cuda", seed=3))
    return model


def _prefill(model, cache, lens, page, max_blocks, seed):
    """Prefill ``len(lens)`` text sequences through the ordinary path; returns their block tables."""
    g = torch.Generator().manual_seed(seed)
    V = model.arch.text.vocab_size
    B = len(lens)
    bt = torch.full((B, max_blocks), -1, dtype=torch.int32)
    nxt = 0
    ids, pos, slots, cu = [], [], [], [0]
    for b, n in enumerate(lens):
        pages = -(-(n + 2) // page)  # room for two decode tokens too
        bt[b, :pages] = torch.arange(nxt, nxt + pages, dtype=torch.int32)
        nxt += pages
        ids.append(torch.randint(0, V, (n,), generator=g))
        pos.append(torch.arange(n, dtype=torch.int32))
        slots.append(torch.tensor([int(bt[b, j // page]) * page + j % page for j in range(n)], dtype=torch.int64))
        cu.append(cu[-1] + n)
    ids, p1, slots = torch.cat(ids).cuda(), torch.cat(pos), torch.cat(slots).cuda()
    positions = torch.stack([p1, p1, p1]).contiguous().cuda()
    meta = AttnMeta(is_prefill=True, block_tables=bt.cuda(), slots=slots, cu_seqlens_q=torch.tensor(cu, dtype=torch.int32).cuda(),
                    kv_lens=torch.tensor(lens, dtype=torch.int32).cuda(), max_q_len=max(lens), no_history=True)
    model.forward(ids, positions, meta, cache)
    return bt


def _decode_inputs(model, bt, lens, page, seed, pad_to):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    T = pad_to
    ids = torch.zeros(T, dtype=torch.int64)
    ids[:B] = torch.randint(0, model.arch.text.vocab_size, (B,), generator=g)
    pos = torch.zeros((3, T), dtype=torch.int32)
    slots = torch.full((T,), -1, dtype=torch.int64)
    ctx = torch.zeros(T, dtype=torch.int32)
    table = torch.full((T, bt.shape[1]), -1, dtype=torch.int32)
    for b, n in enumerate(lens):
        pos[:, b] = n
        slots[b] = int(bt[b, n // page]) * page + n % page
        ctx[b] = n + 1
        table[b] = bt[b]
    return ids.cuda(), pos.cuda(), slots.cuda(), ctx.cuda(), table.cuda()


@pytest.mark.parametrize("arch_name,mode,lens,pad_to", [
    ("tiny", ops.KV_FP8_SCALED, (37,), 1),
    ("tiny", ops.KV_BF16, (5, 300, 64), 4),
    ("tiny", ops.KV_FP8_SCALED, (383, 129), 2),       # several staged chunks per split
    ("8b2", ops.KV_FP8_SCALED, (700,), 1),
    ("8b2", ops.KV_FP8_SCALED, (1500,), 1),
    ("8b2", ops.KV_FP8_SCALED, (255, 1, 513), 4),     # one padded row
    ("8b2", ops.KV_FP8_SCALED, (1400, 90, 256, 1279), 4),
    ("8b2", ops.KV_BF16, (130, 40), 2),
    ("8b2", ops.KV_BF16, (1000,), 1),
    ("8b2", ops.KV_FP8, (300, 1100, 7), 4),
])
def test_persistent_decode_matches_the_per_layer_chain(cuda_device, monkeypatch, arch_name, mode, lens, pad_to):
    arch = Qwen3VLArch.tiny() if arch_name == "tiny" else Qwen3VLArch.qwen3_vl_8b_2layer()
    t = arch.text
    page = 256 if arch_name != "tiny" else 64
    max_blocks = 8
    model = _model(arch)
    blocks = sum(-(-(n + 2) // page) for n in lens) + 1
    cache_a = ops.KVCache(t.num_layers, blocks, t.num_kv_heads, page, t.head_dim, mode, "cuda")
    bt = _prefill(model, cache_a, lens, page, max_blocks, seed=11)
    cache_b = ops.KVCache(t.num_layers, blocks, t.num_kv_heads, page, t.head_dim, mode, "cuda")
    cache_b.payload.copy_(cache_a.payload)
    if cache_a.scales is not None:
        cache_b.scales.copy_(cache_a.scales)
    ids, pos, slots, ctx, table = _decode_inputs(model, bt, lens, page, seed=12, pad_to=pad_to)

    def step(cache, enabled):
        monkeypatch.setattr(dl, "ENABLED", enabled)
        meta = AttnMeta(is_prefill=False, block_tables=table, slots=slots, context_lens=ctx,
                        nsplit=ops.decode_splits(pad_to, t.num_kv_heads))
        h = model.forward(ids, pos, meta, cache).clone()
        torch.cuda.synchronize()
        native.check_status()
        return h

    want = step(cache_a, False)
    got = step(cache_b, True)
    assert model._decode_plan(cache_b, pad_to) is not None
    B = len(lens)
    # hidden states after the final norm have unit scale; both paths round to bf16 at different points
    diff = (got[:B].float() - want[:B].float()).abs()
    assert diff.max() < 0.25 and diff.mean() < 0.02, (float(diff.max()), float(diff.mean()))
    # the K / V rows of the new tokens: same pages, same values up to one quantisation step
    ka, kb = cache_a.dequant(0, t.num_layers - 1), cache_b.dequant(0, t.num_layers - 1)
    va, vb = cache_a.dequant(1, 0), cache_b.dequant(1, 0)
    for b, n in enumerate(lens):
        blk, off = int(bt[b, n // page]), n % page
        for x, y in ((ka, kb), (va, vb)):
            rows_a, rows_b = x[blk, :, off], y[blk, :, off]
            scale = rows_a.abs().max().clamp_min(1e-3)
            assert ((rows_a - rows_b).abs().max() / scale) < 0.15, (b, float((rows_a - rows_b).abs().max()), float(scale))
    # nothing but the new rows changed
    changed = (cache_a.payload.float() != cache_b.payload.float()).any(dim=-1)  # [2, L, blocks, Hkv, page]
    changed = changed.any(dim=3).any(dim=1).any(dim=0)                          # [blocks, page]
    for b, n in enumerate(lens):
        changed[int(bt[b, n // page]), n % page] = False
    assert not bool(changed.any())


def test_persistent_decode_second_step_reads_the_first_steps_rows(cuda_device, monkeypatch):
    """Two consecutive steps of one sequence (the second attends over the row the first stored) and
    replay from a CUDA graph give the same hidden states as eager launches."""
    arch = Qwen3VLArch.qwen3_vl_8b_2layer()
    t = arch.text
    page, max_blocks, lens = 256, 4, (255,)
    model = _model(arch)
    cache = ops.KVCache(t.num_layers, 4, t.num_kv_heads, page, t.head_dim, ops.KV_FP8_SCALED, "cuda")
    bt = _prefill(model, cache, lens, page, max_blocks, seed=21)
    snapshot = (cache.payload.clone(), cache.scales.clone())
    monkeypatch.setattr(dl, "ENABLED", True)

    def two_steps(run):
        cache.payload.copy_(snapshot[0])
        cache.scales.copy_(snapshot[1])
        outs = []
        for k in range(2):
            ids, pos, slots, ctx, table = _decode_inputs(model, bt, (lens[0] + k,), page, seed=30 + k, pad_to=1)
            outs.append(run(ids, pos, slots, ctx, table))
        torch.cuda.synchronize()
        return outs

    def eager(ids, pos, slots, ctx, table):
        meta = AttnMeta(is_prefill=False, block_tables=table, slots=slots, context_lens=ctx)
        return model.forward(ids, pos, meta, cache).clone()

    first = two_steps(eager)
    # graph replay with static input buffers
    s_ids, s_pos, s_slots, s_ctx, s_table = _decode_inputs(model, bt, lens, page, seed=30, pad_to=1)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        meta = AttnMeta(is_prefill=False, block_tables=s_table, slots=s_slots, context_lens=s_ctx)
        model.forward(s_ids, s_pos, meta, cache)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = model.forward(s_ids, s_pos, meta, cache)
    torch.cuda.current_stream().wait_stream(stream)

    def replay(ids, pos, slots, ctx, table):
        for dst, src in ((s_ids, ids), (s_pos, pos), (s_slots, slots), (s_ctx, ctx), (s_table, table)):
            dst.copy_(src)
        graph.replay()
        return out.clone()

    second = two_steps(replay)
    native.check_status()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    assert not torch.equal(first[0], first[1])


def test_sequence_numbers_wrap_without_a_stale_word_being_taken(cuda_device, monkeypatch):
    """The hand-off words carry 32-bit sequence numbers.  Steps taken while the base passes the end
    of the number space give the same result as before: the base starts over, the wrap
    generation grows and the plan's word buffers are zeroed first."""
    arch = Qwen3VLArch.tiny()
    t = arch.text
    page, max_blocks, lens = 64, 4, (100, 7)
    model = _model(arch)
    cache = ops.KVCache(t.num_layers, 5, t.num_kv_heads, page, t.head_dim, ops.KV_FP8_SCALED, "cuda")
    bt = _prefill(model, cache, lens, page, max_blocks, seed=5)
    snapshot = (cache.payload.clone(), cache.scales.clone())
    monkeypatch.setattr(dl, "ENABLED", True)
    ids, pos, slots, ctx, table = _decode_inputs(model, bt, lens, page, seed=6, pad_to=2)
    meta = AttnMeta(is_prefill=False, block_tables=table, slots=slots, context_lens=ctx)

    def step():
        cache.payload.copy_(snapshot[0])
        cache.scales.copy_(snapshot[1])
        h = model.forward(ids, pos, meta, cache).clone()
        torch.cuda.synchronize()
        native.check_status()
        return h

    want = step()
    state = model._decode_plan(cache, 2).state
    seq_step = int(native.lib().prism_decode_layers_seq_step(t.num_layers))
    generation = int(state[1])
    state[0] = 0xFFFFFFFF - 4 * seq_step - 3
    for _ in range(8):
        assert torch.equal(step(), want)
    assert int(state[1]) == generation + 1 and int(state[0]) < 16 * seq_step
