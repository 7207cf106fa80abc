"""Module-level building blocks: every class against plain PyTorch arithmetic; the
tensor-parallel ones with all ranks built side by side in one process (their partial results
are summed / gathered by a small in-process communicator)."""

import math

import pytest
import torch
import torch.nn.functional as F

from prism_infer_b200 import layers, ops
from prism_infer_b200.models.qwen3_vl import AttnMeta, TPComm


class _Ranks:
    """In-process stand-in for the collectives: ranks call in order 0..n-1, the last one's call
    completes the exchange and every rank reads the result afterwards."""

    def __init__(self, size):
        self.size = size
        self.comms = [self._Comm(self, r) for r in range(size)]
        self.pending = []

    class _Comm(TPComm):
        def __init__(self, owner, rank):
            self.owner, self.rank, self.size = owner, rank, owner.size

        def reduce_dense(self, x):
            self.owner.pending.append(x)
            return x

        def gather_logits(self, x):
            self.owner.pending.append(x)
            return x

        def greedy_merge(self, val, ids):
            self.owner.pending.append((val, ids))
            return ids

    def take(self):
        out, self.pending = self.pending, []
        return out


def test_rmsnorm_silu_rotary_match_plain_arithmetic():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 5, 64, generator=g)
    res = torch.randn(3, 5, 64, generator=g)
    norm = layers.RMSNorm(64, eps=1e-5)
    norm.weight.data = 1 + 0.1 * torch.randn(64, generator=g)
    want = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * norm.weight
    assert torch.allclose(norm(x), want, atol=1e-5)
    keep = res.clone()
    y, new_res = norm(x, res)
    s = x + res
    assert torch.equal(res, keep), "the caller's residual is not modified"
    assert torch.allclose(new_res, s, atol=1e-6)
    assert torch.allclose(y, s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * norm.weight, atol=1e-5)

    gu = torch.randn(2, 7, 48, generator=g)
    assert torch.allclose(layers.SiluAndMul()(gu), F.silu(gu[..., :24]) * gu[..., 24:], atol=1e-6)
    with pytest.raises(ValueError):
        layers.SiluAndMul()(torch.zeros(2, 5))

    rope = layers.get_rope(32, 32, 128, 10000.0)
    assert rope is layers.get_rope(32, 32, 128, 10000.0)
    pos = torch.tensor([0, 3, 77])
    q = torch.randn(3, 4, 32, generator=g)
    k = torch.randn(3, 2, 32, generator=g)
    rq, rk = rope(pos, q, k)
    inv = 1.0 / 10000.0 ** (torch.arange(0, 32, 2).float() / 32)
    ang = pos[:, None].float() * inv[None]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    want_q = torch.cat((q[..., :16] * cos - q[..., 16:] * sin, q[..., 16:] * cos + q[..., :16] * sin), -1)
    assert torch.allclose(rq, want_q, atol=1e-5) and torch.equal(rq[0], q[0]) and rk.shape == k.shape
    for bad in [(32, 16, 128, 1e4), (31, 31, 128, 1e4), (32, 32, 0, 1e4), (32, 32, 8, -1.0), (True, 32, 8, 1e4)]:
        with pytest.raises(ValueError):
            layers.RotaryEmbedding(*bad)
    with pytest.raises(NotImplementedError):
        layers.get_rope(32, 32, 128, 1e4, {"type": "yarn"})


def test_divide_rejects_bad_dimensions():
    assert layers.divide(12, 4) == 3 and layers.divide(0, 2) == 0
    for a, b in [(10, 4), (-2, 2), (4, 0), (True, 1), (4.0, 2)]:
        with pytest.raises(ValueError):
            layers.divide(a, b)


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_tensor_parallel_mlp_and_attention_projections_match_full_weights(tp):
    """QKV (packed, grouped-query) -> row-parallel output and merged gate/up -> SwiGLU ->
    row-parallel down, loaded from full checkpoint tensors through ``weight_loader``."""
    g = torch.Generator().manual_seed(tp)
    H, D, Hq, Hkv, I = 64, 16, 8, 4, 96
    full = {n: torch.randn(*s, generator=g) * 0.1 for n, s in
            dict(q=(Hq * D, H), k=(Hkv * D, H), v=(Hkv * D, H), qb=(Hq * D,), kb=(Hkv * D,), vb=(Hkv * D,), o=(H, Hq * D), ob=(H,),
                 gate=(I, H), up=(I, H), down=(H, I)).items()}
    x = torch.randn(2, 5, H, generator=g)
    ranks = _Ranks(tp)
    outs_attn, outs_mlp, qkv_parts = [], [], []
    for comm in ranks.comms:
        qkv = layers.QKVParallelLinear(H, D, Hq, Hkv, bias=True, comm=comm)
        for s in "qkv":
            qkv.weight.weight_loader(qkv.weight, full[s], s)
            qkv.bias.weight_loader(qkv.bias, full[s + "b"], s)
        o = layers.RowParallelLinear(Hq * D, H, bias=True, comm=comm)
        o.weight.weight_loader(o.weight, full["o"])
        o.bias.weight_loader(o.bias, full["ob"])
        gate_up = layers.MergedColumnParallelLinear(H, [I, I], comm=comm)
        gate_up.weight.weight_loader(gate_up.weight, full["gate"], 0)
        gate_up.weight.weight_loader(gate_up.weight, full["up"], 1)
        down = layers.RowParallelLinear(I, H, comm=comm)
        down.weight.weight_loader(down.weight, full["down"])
        assert qkv.weight.shape == ((Hq + 2 * Hkv) * D // tp, H) and down.weight.shape == (H, I // tp)
        y = qkv(x)
        qkv_parts.append(y)
        outs_attn.append(o(y[..., : Hq * D // tp]))  # "attention" = identity on the query part
        outs_mlp.append(down(layers.SiluAndMul()(gate_up(x))))
    want_q = F.linear(x, full["q"], full["qb"])
    got_q = torch.cat([p[..., : Hq * D // tp] for p in qkv_parts], -1)
    got_v = torch.cat([p[..., (Hq + Hkv) * D // tp:] for p in qkv_parts], -1)
    assert torch.allclose(got_q, want_q, atol=1e-5)
    assert torch.allclose(got_v, F.linear(x, full["v"], full["vb"]), atol=1e-5)
    assert torch.allclose(sum(outs_attn), F.linear(want_q, full["o"], full["ob"]), atol=1e-4)
    want_mlp = F.linear(F.silu(F.linear(x, full["gate"])) * F.linear(x, full["up"]), full["down"])
    assert torch.allclose(sum(outs_mlp), want_mlp, atol=1e-4)
    with pytest.raises(ValueError):
        qkv.weight_loader(qkv.weight, full["q"], "x")
    with pytest.raises(ValueError):
        gate_up.weight_loader(gate_up.weight, full["gate"], 2)
    with pytest.raises(ValueError):
        layers.ColumnParallelLinear(8, 6, comm=ranks.comms[0]) if tp == 4 else layers.divide(3, 2)
    rep = layers.ReplicatedLinear(H, 8, bias=True)
    rep.weight.weight_loader(rep.weight, full["q"][:8])
    rep.bias.weight_loader(rep.bias, full["qb"][:8])
    assert torch.allclose(rep(x), F.linear(x, full["q"][:8], full["qb"][:8]), atol=1e-5)


@pytest.mark.parametrize("tp", [1, 4])
def test_vocab_parallel_embedding_and_head(tp):
    g = torch.Generator().manual_seed(7)
    V, H = 64, 32
    table = torch.randn(V, H, generator=g)
    head_w = torch.randn(V, H, generator=g)
    ids = torch.randint(0, V, (2, 9), generator=g)
    x = torch.randn(11, H, generator=g)
    last = torch.tensor([3, 10])
    ranks = _Ranks(tp)
    emb_parts, logit_parts, greedy_parts = [], [], []
    for comm in ranks.comms:
        emb = layers.VocabParallelEmbedding(V, H, comm=comm)
        emb.weight.weight_loader(emb.weight, table)
        head = layers.ParallelLMHead(V, H, comm=comm)
        head.weight.weight_loader(head.weight, head_w)
        emb_parts.append(emb(ids))
        out = head(x, last)
        assert (out is None) == (tp > 1 and comm.rank > 0)
        logit_parts.append(head._local_logits(x[last]))
        toks = head.compute_greedy_tokens(x, last)
        greedy_parts.append(ranks.take()[-1] if tp > 1 else toks)
    assert torch.allclose(sum(emb_parts), table[ids], atol=1e-6)
    want_logits = F.linear(x[last], head_w)
    assert torch.allclose(torch.cat(logit_parts, -1), want_logits, atol=1e-5)
    if tp == 1:
        assert torch.equal(greedy_parts[0], want_logits.argmax(-1))
    else:
        vals = torch.stack([v for v, _ in greedy_parts])
        idx = torch.stack([i for _, i in greedy_parts])
        assert torch.equal(idx.gather(0, vals.argmax(0, keepdim=True))[0], want_logits.argmax(-1))
    with pytest.raises(ValueError):
        layers.ParallelLMHead(V, H, bias=True)
    with pytest.raises(TypeError):
        layers.ParallelLMHead(V, H, select_prefill_tokens=1)
    with pytest.raises(ValueError):
        layers.VocabParallelEmbedding(0, H)


def test_sampler_modes():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(6, 50, generator=g)
    s = layers.Sampler(seed=5)
    assert torch.equal(s(logits, None, sampling_mode="greedy"), logits.argmax(-1))
    assert torch.equal(s(logits, torch.zeros(6)), logits.argmax(-1))
    with pytest.raises(ValueError):
        s(logits, None)
    with pytest.raises(ValueError):
        s(logits, torch.ones(6), sampling_mode="beam")
    temps = torch.tensor([0.0, 1.0, 0.0, 0.5, 0.0, 2.0])
    mixed = s(logits, temps)
    assert torch.equal(mixed[temps == 0], logits.argmax(-1)[temps == 0])
    # a peaked distribution is sampled at its peak; a flat one visits several tokens over calls
    peaked = torch.full((4, 50), -30.0)
    peaked[:, 17] = 30.0
    assert torch.equal(s(peaked, torch.ones(4), sampling_mode="random"), torch.full((4,), 17))
    seen = {int(s(torch.zeros(1, 50), torch.ones(1), sampling_mode="random")) for _ in range(24)}
    assert len(seen) > 4


def _meta_prefill(T, cache_blocks, page):
    slots = torch.arange(T, dtype=torch.int64)
    bt = torch.arange(cache_blocks, dtype=torch.int32)[None]
    return AttnMeta(True, bt, slots, cu_seqlens_q=torch.tensor([0, T], dtype=torch.int32), kv_lens=torch.tensor([T], dtype=torch.int32),
                    max_q_len=T, no_history=True)


def _attention_reference(q, k, v, causal_offset):
    T, Hq, D = q.shape
    G = Hq // k.shape[1]
    kk, vv = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
    s = torch.einsum("thd,shd->hts", q.float(), kk.float()) / math.sqrt(D)
    S = k.shape[0]
    mask = torch.arange(S)[None, :] > (torch.arange(T)[:, None] + causal_offset)
    s = s.masked_fill(mask[None], float("-inf"))
    return torch.einsum("hts,shd->thd", s.softmax(-1), vv.float())


def test_attention_router_prefill_then_decode_cpu():
    g = torch.Generator().manual_seed(11)
    Hq, Hkv, D, page, T = 4, 2, 16, 8, 13
    cache = ops.KVCache(1, 4, Hkv, page, D, ops.KV_BF16, "cpu", dtype=torch.float32)
    attn = layers.Attention(Hq, D, D ** -0.5, Hkv)
    attn.bind_cache(cache, 0)
    q = torch.randn(T, Hq * D, generator=g)
    k = torch.randn(T, Hkv * D, generator=g)
    v = torch.randn(T, Hkv * D, generator=g)
    out = attn(q, k, v, _meta_prefill(T, 4, page))
    want = _attention_reference(q.view(T, Hq, D), k.view(T, Hkv, D), v.view(T, Hkv, D), 0)
    assert torch.allclose(out.view(T, Hq, D), want, atol=1e-4)
    # the same chunk again as a "later chunk": it reads the pages the first call stored
    meta = _meta_prefill(T, 4, page)
    meta.no_history = False
    assert torch.allclose(attn(q, k, v, meta).view(T, Hq, D), want, atol=1e-4)
    # one decode step at position T
    q1 = torch.randn(1, Hq * D, generator=g)
    k1 = torch.randn(1, Hkv * D, generator=g)
    v1 = torch.randn(1, Hkv * D, generator=g)
    dmeta = AttnMeta(False, torch.arange(4, dtype=torch.int32)[None], torch.tensor([T]), context_lens=torch.tensor([T + 1], dtype=torch.int32))
    got = attn(q1, k1, v1, dmeta)
    allk = torch.cat((k, k1)).view(T + 1, Hkv, D)
    allv = torch.cat((v, v1)).view(T + 1, Hkv, D)
    assert torch.allclose(got.view(1, Hq, D), _attention_reference(q1.view(1, Hq, D), allk, allv, T), atol=1e-4)
    with pytest.raises(ValueError):
        layers.Attention(6, 16, None, 4)
    with pytest.raises(ValueError):
        layers.Attention(4, 16, 1.0, 2)


@pytest.mark.gpu
def test_layers_run_the_cuda_kernels(cuda_device):
    """bf16 modules on the device against fp32 arithmetic on the host."""
    g = torch.Generator().manual_seed(0)
    H, I, T = 1024, 3072, 48
    x = torch.randn(T, H, generator=g)
    res = torch.randn(T, H, generator=g)
    norm = layers.RMSNorm(H).to("cuda", torch.bfloat16)
    y, new_res = norm(x.cuda().bfloat16(), res.cuda().bfloat16())
    s = (x.bfloat16().float() + res.bfloat16().float())
    assert (new_res.float().cpu() - s).abs().max() < 4e-2
    assert (y.float().cpu() - s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6)).abs().max() < 6e-2
    gate_up = layers.MergedColumnParallelLinear(H, [I, I]).to("cuda", torch.bfloat16)
    down = layers.RowParallelLinear(I, H).to("cuda", torch.bfloat16)
    wg = torch.randn(I, H, generator=g) * H ** -0.5
    wu = torch.randn(I, H, generator=g) * H ** -0.5
    wd = torch.randn(H, I, generator=g) * I ** -0.5
    gate_up.weight.weight_loader(gate_up.weight, wg, 0)
    gate_up.weight.weight_loader(gate_up.weight, wu, 1)
    down.weight.weight_loader(down.weight, wd)
    out = down(layers.SiluAndMul()(gate_up(x.cuda().bfloat16()))).float().cpu()
    xb = x.bfloat16().float()
    want = F.linear(F.silu(F.linear(xb, wg.bfloat16().float())) * F.linear(xb, wu.bfloat16().float()), wd.bfloat16().float())
    assert (out - want).abs().max() < 5e-2 * max(1.0, want.abs().max().item())
    head = layers.ParallelLMHead(4096, H).to("cuda", torch.bfloat16)
    hw = torch.randn(4096, H, generator=g) * H ** -0.5
    head.weight.weight_loader(head.weight, hw)
    toks = head.compute_greedy_tokens(x.cuda().bfloat16())
    logits = F.linear(xb, hw.bfloat16().float())
    picked = logits.gather(1, toks.cpu()[:, None])[:, 0]
    assert (logits.max(-1).values - picked).max() < 2e-2  # the arg-max up to bf16 rounding of near-ties
    assert torch.equal(layers.Sampler()(logits.cuda(), None, sampling_mode="greedy").cpu(), logits.argmax(-1))
    ops.native.check_status()


def test_decoder_composed_of_the_layer_modules_matches_the_oracle():
    """The module building blocks are not on the engine's hot path, so nothing else notices if they drift from it.
    A two-layer text decoder put together from them (weights loaded through their loaders from checkpoint names)
    must give the oracle's hidden states: a prefill chunk, a second chunk over the paged cache, then a decode step."""
    from prism_infer_b200 import ops
    from prism_infer_b200.layers import (Attention, MergedColumnParallelLinear, QKVParallelLinear, RMSNorm, RowParallelLinear, SiluAndMul,
                                         VocabParallelEmbedding, get_rope)
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.qwen3_vl import AttnMeta
    from prism_infer_b200.models.reference_model import ReferenceQwen3VL
    from prism_infer_b200.models.weights import random_weights

    arch = Qwen3VLArch.tiny()
    t = arch.text
    w = random_weights(arch, dtype=torch.float32, seed=0)
    oracle = ReferenceQwen3VL(arch, w)
    lm = "model.language_model"

    class Layer(torch.nn.Module):
        def __init__(self, i):
            super().__init__()
            p = f"{lm}.layers.{i}"
            self.input_norm, self.post_norm = RMSNorm(t.hidden_size, t.rms_norm_eps), RMSNorm(t.hidden_size, t.rms_norm_eps)
            self.q_norm, self.k_norm = RMSNorm(t.head_dim, t.rms_norm_eps), RMSNorm(t.head_dim, t.rms_norm_eps)
            self.qkv = QKVParallelLinear(t.hidden_size, t.head_dim, t.num_heads, t.num_kv_heads)
            self.o = RowParallelLinear(t.num_heads * t.head_dim, t.hidden_size)
            self.gate_up = MergedColumnParallelLinear(t.hidden_size, [t.intermediate_size, t.intermediate_size])
            self.down = RowParallelLinear(t.intermediate_size, t.hidden_size)
            self.act, self.attn = SiluAndMul(), Attention(t.num_heads, t.head_dim, num_kv_heads=t.num_kv_heads, layer=i)
            self.rope = get_rope(t.head_dim, t.head_dim, 512, t.rope_theta)
            for name, mod in (("input_layernorm", self.input_norm), ("post_attention_layernorm", self.post_norm),
                              ("self_attn.q_norm", self.q_norm), ("self_attn.k_norm", self.k_norm)):
                mod.weight.data.copy_(w[f"{p}.{name}.weight"])
            for shard in "qkv":
                self.qkv.weight_loader(self.qkv.weight, w[f"{p}.self_attn.{shard}_proj.weight"], shard)
            self.o.weight_loader(self.o.weight, w[f"{p}.self_attn.o_proj.weight"])
            self.gate_up.weight_loader(self.gate_up.weight, w[f"{p}.mlp.gate_proj.weight"], 0)
            self.gate_up.weight_loader(self.gate_up.weight, w[f"{p}.mlp.up_proj.weight"], 1)
            self.down.weight_loader(self.down.weight, w[f"{p}.mlp.down_proj.weight"])

        def forward(self, x, positions, meta):
            n = x.shape[0]
            q, k, v = self.qkv(self.input_norm(x)).split([t.num_heads * t.head_dim, t.num_kv_heads * t.head_dim, t.num_kv_heads * t.head_dim], dim=-1)
            q = self.q_norm(q.reshape(n, t.num_heads, t.head_dim))
            k = self.k_norm(k.reshape(n, t.num_kv_heads, t.head_dim))
            q, k = self.rope(positions, q, k)
            x = x + self.o(self.attn(q.reshape(n, -1), k.reshape(n, -1), v, meta))
            return x + self.down(self.act(self.gate_up(self.post_norm(x))))

    embed = VocabParallelEmbedding(t.vocab_size, t.hidden_size)
    embed.weight_loader(embed.weight, w[f"{lm}.embed_tokens.weight"])
    final = RMSNorm(t.hidden_size, t.rms_norm_eps)
    final.weight.data.copy_(w[f"{lm}.norm.weight"])
    layers = [Layer(i) for i in range(t.num_layers)]
    page = 16
    cache = ops.KVCache(t.num_layers, 4, t.num_kv_heads, page, t.head_dim, ops.KV_BF16, "cpu", dtype=torch.float32)
    for layer in layers:
        layer.attn.bind_cache(cache)

    ids = torch.randint(0, t.vocab_size, (27,), generator=torch.Generator().manual_seed(3))
    want = oracle.text_forward(ids, torch.arange(27).expand(3, -1))
    bt = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32)

    def run(lo, hi, meta):
        x = embed(ids[lo:hi])
        pos = torch.arange(lo, hi)
        for layer in layers:
            x = layer(x, pos, meta)
        return final(x)

    def slots(lo, hi):
        j = torch.arange(lo, hi)
        return bt[0, (j // page).long()].long() * page + j % page

    def prefill_meta(lo, hi):
        return AttnMeta(is_prefill=True, block_tables=bt, slots=slots(lo, hi), cu_seqlens_q=torch.tensor([0, hi - lo], dtype=torch.int32),
                        kv_lens=torch.tensor([hi], dtype=torch.int32), max_q_len=hi - lo, no_history=lo == 0)

    with torch.no_grad():
        first = run(0, 20, prefill_meta(0, 20))                      # fresh K / V rows
        second = run(20, 26, prefill_meta(20, 26))                   # six tokens over twenty cached ones
        last = run(26, 27, AttnMeta(is_prefill=False, block_tables=bt, slots=slots(26, 27), context_lens=torch.tensor([27], dtype=torch.int32)))
    got = torch.cat((first, second, last))
    assert got.shape == want.shape
    assert float((got - want).abs().max()) < 2e-4, float((got - want).abs().max())
