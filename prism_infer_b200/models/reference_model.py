"""Plain-PyTorch Qwen3-VL forward used as the numerical oracle.

No paging, no fused ops, no custom kernels: dense causal attention over the whole
prompt, recomputed from scratch at every greedy step.  Every engine path (CPU ops,
sm_100a kernels, tensor-parallel ranks) is tested against this forward.  Structure
follows Hugging Face ``Qwen3VLForConditionalGeneration`` as summarised in the
reference's ``prism_infer/models/qwen3_vl.py:832-1022`` (decoder, DeepStack after
layers 0..k-1) and ``prism_infer/vision/vision_encoder.py:107-453,546-740`` (vision
tower, mergers).
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.nn.functional as F

from .architecture import Qwen3VLArch
from .position import (
    mrope_cos_sin,
    rotate_half,
    rope_index,
    vision_patch_coords,
    vision_pos_embed_plan,
    vision_segments,
)
from .weights import LM, VIS


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y.to(x.dtype)) * w


class ReferenceQwen3VL:
    """Stateless functional model over a ``{hf_name: tensor}`` dictionary."""

    def __init__(self, arch: Qwen3VLArch, weights: dict[str, torch.Tensor]):
        self.arch = arch
        self.w = weights
        any_w = next(iter(weights.values()))
        self.dtype = any_w.dtype
        self.device = any_w.device

    # ------------------------------------------------------------------ vision
    def vision(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]]):
        """``pixel_values [N, C*Tp*P*P]`` -> ``(main [N/4, H], [deepstack_k [N/4, H]])``."""
        v, w = self.arch.vision, self.w
        grid = [tuple(int(x) for x in row) for row in (grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else grid_thw)]
        x = pixel_values.to(self.dtype)
        pw = w[f"{VIS}.patch_embed.proj.weight"].reshape(v.hidden_size, -1)
        x = F.linear(x, pw, w[f"{VIS}.patch_embed.proj.bias"])
        idx, wt = vision_pos_embed_plan(grid, v.grid_per_side, v.spatial_merge_size)
        table = w[f"{VIS}.pos_embed.weight"]
        pos = (table[idx.to(self.device)].float() * wt.to(self.device)[:, :, None]).sum(0)
        x = x + pos.to(self.dtype)

        hd = v.head_dim
        quarter = hd // 4
        inv = 1.0 / (v.rope_theta ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))
        rc = vision_patch_coords(grid, v.spatial_merge_size).float()
        ang = torch.cat((rc[:, 0:1] * inv[None, :], rc[:, 1:2] * inv[None, :]), dim=-1)  # [N, hd/2]
        assert ang.shape[1] == 2 * quarter
        ang = torch.cat((ang, ang), dim=-1).to(self.device)
        cos, sin = ang.cos(), ang.sin()
        segs = vision_segments(grid)

        deep: list[torch.Tensor] = []
        for i in range(v.depth):
            b = f"{VIS}.blocks.{i}"
            h = F.layer_norm(x, (v.hidden_size,), w[f"{b}.norm1.weight"], w[f"{b}.norm1.bias"], v.layer_norm_eps)
            qkv = F.linear(h, w[f"{b}.attn.qkv.weight"], w[f"{b}.attn.qkv.bias"])
            n = qkv.shape[0]
            q, k, val = qkv.view(n, 3, v.num_heads, hd).unbind(1)

            def rope(t: torch.Tensor) -> torch.Tensor:
                tf = t.float()
                return (tf * cos[:, None, :] + rotate_half(tf) * sin[:, None, :]).to(t.dtype)

            q, k = rope(q), rope(k)
            outs = []
            start = 0
            for length in segs:
                sl = slice(start, start + length)
                o = F.scaled_dot_product_attention(
                    q[sl].transpose(0, 1).unsqueeze(0).float(),
                    k[sl].transpose(0, 1).unsqueeze(0).float(),
                    val[sl].transpose(0, 1).unsqueeze(0).float(),
                )
                outs.append(o.squeeze(0).transpose(0, 1).reshape(length, -1).to(self.dtype))
                start += length
            a = torch.cat(outs, dim=0)
            x = x + F.linear(a, w[f"{b}.attn.proj.weight"], w[f"{b}.attn.proj.bias"])
            h = F.layer_norm(x, (v.hidden_size,), w[f"{b}.norm2.weight"], w[f"{b}.norm2.bias"], v.layer_norm_eps)
            h = F.gelu(F.linear(h, w[f"{b}.mlp.linear_fc1.weight"], w[f"{b}.mlp.linear_fc1.bias"]), approximate="tanh")
            x = x + F.linear(h, w[f"{b}.mlp.linear_fc2.weight"], w[f"{b}.mlp.linear_fc2.bias"])
            if i in v.deepstack_visual_indexes:
                k_idx = v.deepstack_visual_indexes.index(i)
                deep.append(self._merger(x, f"{VIS}.deepstack_merger_list.{k_idx}", post_norm=True))
        main = self._merger(x, f"{VIS}.merger", post_norm=False)
        return main, deep

    def _merger(self, x: torch.Tensor, prefix: str, *, post_norm: bool) -> torch.Tensor:
        v, w = self.arch.vision, self.w
        if post_norm:
            x = x.reshape(-1, v.merged_dim)
            x = F.layer_norm(x, (v.merged_dim,), w[f"{prefix}.norm.weight"], w[f"{prefix}.norm.bias"], v.layer_norm_eps)
        else:
            x = F.layer_norm(x, (v.hidden_size,), w[f"{prefix}.norm.weight"], w[f"{prefix}.norm.bias"], v.layer_norm_eps)
            x = x.reshape(-1, v.merged_dim)
        x = F.gelu(F.linear(x, w[f"{prefix}.linear_fc1.weight"], w[f"{prefix}.linear_fc1.bias"]))
        return F.linear(x, w[f"{prefix}.linear_fc2.weight"], w[f"{prefix}.linear_fc2.bias"])

    # -------------------------------------------------------------------- text
    def text_forward(
        self,
        input_ids: torch.Tensor,
        positions: torch.Tensor,
        visual: torch.Tensor | None = None,
        deepstack: Sequence[torch.Tensor] | None = None,
    ) -> torch.Tensor:
        """``input_ids [S]``, ``positions [3, S]`` -> hidden ``[S, H]`` after the final norm."""
        t, w = self.arch.text, self.w
        ids = input_ids.to(self.device)
        x = w[f"{LM}.embed_tokens.weight"][ids]
        vmask = (ids == self.arch.image_token_id) | (ids == self.arch.video_token_id)
        if visual is not None:
            x = x.clone()
            x[vmask] = visual.to(x.dtype)
        cos, sin = mrope_cos_sin(positions.to(self.device), t.head_dim, t.rope_theta, t.mrope_section)
        s = ids.shape[0]
        group = t.num_heads // t.num_kv_heads
        for i in range(t.num_layers):
            p = f"{LM}.layers.{i}"
            h = rms_norm(x, w[f"{p}.input_layernorm.weight"], t.rms_norm_eps)
            q = F.linear(h, w[f"{p}.self_attn.q_proj.weight"]).view(s, t.num_heads, t.head_dim)
            k = F.linear(h, w[f"{p}.self_attn.k_proj.weight"]).view(s, t.num_kv_heads, t.head_dim)
            v = F.linear(h, w[f"{p}.self_attn.v_proj.weight"]).view(s, t.num_kv_heads, t.head_dim)
            q = rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], t.rms_norm_eps)
            k = rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], t.rms_norm_eps)

            def rope(z: torch.Tensor) -> torch.Tensor:
                zf = z.float()
                return (zf * cos[:, None, :] + rotate_half(zf) * sin[:, None, :]).to(z.dtype)

            q, k = rope(q), rope(k)
            o = F.scaled_dot_product_attention(
                q.transpose(0, 1).unsqueeze(0).float(),
                k.repeat_interleave(group, dim=1).transpose(0, 1).unsqueeze(0).float(),
                v.repeat_interleave(group, dim=1).transpose(0, 1).unsqueeze(0).float(),
                is_causal=True,
            )
            o = o.squeeze(0).transpose(0, 1).reshape(s, -1).to(x.dtype)
            x = x + F.linear(o, w[f"{p}.self_attn.o_proj.weight"])
            h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], t.rms_norm_eps)
            g = F.linear(h, w[f"{p}.mlp.gate_proj.weight"])
            u = F.linear(h, w[f"{p}.mlp.up_proj.weight"])
            x = x + F.linear(F.silu(g) * u, w[f"{p}.mlp.down_proj.weight"])
            if deepstack is not None and i < len(deepstack):
                x = x.clone()
                x[vmask] = x[vmask] + deepstack[i].to(x.dtype)
        return rms_norm(x, w[f"{LM}.norm.weight"], t.rms_norm_eps)

    def lm_head(self, hidden: torch.Tensor) -> torch.Tensor:
        name = "lm_head.weight" if "lm_head.weight" in self.w else f"{LM}.embed_tokens.weight"
        return F.linear(hidden, self.w[name]).float()

    # ---------------------------------------------------------------- generate
    @torch.no_grad()
    def logits(
        self,
        input_ids: Sequence[int],
        *,
        pixel_values: torch.Tensor | None = None,
        image_grid_thw=None,
        video_grid_thw=None,
    ) -> torch.Tensor:
        """Full-sequence logits ``[S, V]`` (fp32)."""
        ids = torch.tensor(list(input_ids), dtype=torch.long)
        pos, _ = rope_index(
            ids,
            image_grid_thw=image_grid_thw,
            video_grid_thw=video_grid_thw,
            image_token_id=self.arch.image_token_id,
            video_token_id=self.arch.video_token_id,
            spatial_merge_size=self.arch.vision.spatial_merge_size,
        )
        visual = deep = None
        if pixel_values is not None:
            grids = []
            for g in (image_grid_thw, video_grid_thw):
                if g is not None:
                    grids.extend(g.tolist() if isinstance(g, torch.Tensor) else g)
            visual, deep = self.vision(pixel_values.to(self.device), grids)
        hidden = self.text_forward(ids, pos[:, 0, :], visual, deep)
        return self.lm_head(hidden)

    @torch.no_grad()
    def generate_greedy(
        self,
        input_ids: Sequence[int],
        max_tokens: int,
        *,
        pixel_values: torch.Tensor | None = None,
        image_grid_thw=None,
        video_grid_thw=None,
        return_logits: bool = False,
    ):
        """Greedy decode by full recomputation; the vision tower runs once."""
        ids = list(int(t) for t in input_ids)
        visual = deep = None
        if pixel_values is not None:
            grids = []
            for g in (image_grid_thw, video_grid_thw):
                if g is not None:
                    grids.extend(g.tolist() if isinstance(g, torch.Tensor) else g)
            visual, deep = self.vision(pixel_values.to(self.device), grids)
        prompt_pos, delta = rope_index(
            ids,
            image_grid_thw=image_grid_thw,
            video_grid_thw=video_grid_thw,
            image_token_id=self.arch.image_token_id,
            video_token_id=self.arch.video_token_id,
            spatial_merge_size=self.arch.vision.spatial_merge_size,
        )
        prompt_pos = prompt_pos[:, 0, :]
        out: list[int] = []
        step_logits: list[torch.Tensor] = []
        for _ in range(max_tokens):
            n = len(ids)
            extra = torch.arange(prompt_pos.shape[1], n, dtype=torch.int64) + delta
            pos = torch.cat((prompt_pos, extra.expand(3, -1)), dim=1)
            hidden = self.text_forward(torch.tensor(ids), pos, visual, deep)
            logit = self.lm_head(hidden[-1:])[0]
            step_logits.append(logit.cpu())
            tok = int(torch.argmax(logit).item())
            out.append(tok)
            ids.append(tok)
        if return_logits:
            return out, torch.stack(step_logits)
        return out
