"""Grouped-query causal self-attention over the paged cache.

q = x Wq^T + bq, k = x Wk^T + bk, v = x Wv^T + bv (one fused product on the concatenated
weights), position encoding on q and k, k and v stored to the cache, every row attends to its
request's cached keys (optionally only the last ``window`` of them) with query head h reading kv
head h // (heads / kv_heads), then o = attn Wo^T.  Reference: the ``_attention`` function of
src/mini_llm_runtime/qwen_model_runner.py:75-183 and the decode kernel
csrc/paged_attention_cuda.cu:25-106; the reference keeps q/k/v as three products and has no window.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops import AttentionBatch
from .base import KVCacheNeed, Mixer, TensorSpec, build_part, register_part


class GQAAttention(Mixer):
    graph_safe = True
    supports_norm_fusion = True
    plan_key = "paged_attention"     # every attention layer of a model reads the same work lists

    def __init__(self, spec, compute_dtype):
        super().__init__(spec, compute_dtype)
        a = self.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads = int(a["num_heads"])
        self.num_kv_heads = int(a["num_kv_heads"])
        self.head_dim = int(a["head_dim"])
        self.qkv_bias = bool(a.get("qkv_bias", False))
        self.out_bias = bool(a.get("out_bias", False))
        self.window = a.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("an attention window must be positive")
        self.scale = float(self.head_dim) ** -0.5
        # the position encoding is optional: without one, q and k are used as projected
        self.position = build_part("position", a["position"], compute_dtype) if a.get("position") else None
        self._no_rotation: torch.Tensor | None = None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None
        self.input_norm_eps: float | None = None     # set once the preceding norm's weight is folded in

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, None if self.window is None else int(self.window))

    def tensors(self):
        q_rows = self.num_heads * self.head_dim
        kv_rows = self.num_kv_heads * self.head_dim
        p = self.prefix
        out = {
            p + "q_proj.weight": TensorSpec((q_rows, self.hidden_size)),
            p + "k_proj.weight": TensorSpec((kv_rows, self.hidden_size)),
            p + "v_proj.weight": TensorSpec((kv_rows, self.hidden_size)),
            p + "o_proj.weight": TensorSpec((self.hidden_size, q_rows)),
        }
        if self.qkv_bias:
            out[p + "q_proj.bias"] = TensorSpec((q_rows,), init="bias")
            out[p + "k_proj.bias"] = TensorSpec((kv_rows,), init="bias")
            out[p + "v_proj.bias"] = TensorSpec((kv_rows,), init="bias")
        if self.out_bias:
            out[p + "o_proj.bias"] = TensorSpec((self.hidden_size,), init="bias")
        return out

    def load(self, tensors, device):
        p = self.prefix
        # q, k and v rows stacked so that one product yields [q heads | k heads | v heads].
        self.w_qkv = self._to_compute(
            torch.cat([tensors[p + f"{n}_proj.weight"] for n in "qkv"], dim=0), device)
        if self.qkv_bias:
            self.b_qkv = self._to_compute(
                torch.cat([tensors[p + f"{n}_proj.bias"] for n in "qkv"], dim=0), device)
        self.w_o = self._to_compute(tensors[p + "o_proj.weight"], device)
        if self.out_bias:
            self.b_o = self._to_compute(tensors[p + "o_proj.bias"], device)
        if self.position is not None:
            self.position.load({}, device)
        else:
            self._no_rotation = torch.zeros(self.head_dim // 2, dtype=torch.float32, device=device)

    def absorb_input_norm(self, weight, eps):
        folded = self.w_qkv.float() * weight.to(self.w_qkv.device).float()[None, :]
        self.w_qkv = folded.to(self.compute_dtype).contiguous()
        self.input_norm_eps = float(eps)

    def step_plan(self, host):
        return ops.current().plan_attention(host.lengths, host.position_start)

    def _batch(self, ctx, view) -> AttentionBatch:
        """The step's ragged batch as the attention kernels want it; built once per step and cache
        group and shared by the layers of that group."""
        batch = view.shared.get("attention_batch")
        if batch is None:
            arrays, counts = ctx.plans.get(self.plan_key, ({}, {}))
            batch = AttentionBatch(
                seg_q_start=ctx.seg_q_start, seg_q_len=ctx.seg_q_len, seg_pos0=ctx.seg_pos0, seg_slot=ctx.seg_slot,
                block_table=view.block_table, num_segments=ctx.num_segments, max_q_len=ctx.max_q_len,
                max_kv_len=ctx.max_kv_len, plan=arrays, counts=counts)
            view.shared["attention_batch"] = batch
        return batch

    def forward(self, x, ctx, view, writes_cache, raw_input=False, residual=None):
        """``raw_input``: x is the un-normalised stream and the q/k/v product applies the row scale
        of the folded norm.  ``residual``: the output product adds into it in place."""
        k = ops.current()
        qkv = k.linear(x, self.w_qkv, self.b_qkv, rms_eps=self.input_norm_eps if raw_input else None)
        batch = self._batch(ctx, view)
        frequencies = self._no_rotation if self.position is None else self.position.rotary_frequencies()
        if frequencies is not None:
            # a plain rotary encoding (or none): rotation, cache write and attention may share kernels
            mixed = k.rope_paged_attention(qkv, ctx.positions, frequencies, view.slots, view.k_pool, view.v_pool,
                                           batch, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                                           self.window, writes_cache)
        else:
            q = self.position.rotate_and_store(qkv, ctx, view, self.num_heads, self.num_kv_heads, self.head_dim,
                                               writes_cache)
            mixed = k.paged_attention(q, view.k_pool, view.v_pool, batch, self.num_heads, self.num_kv_heads,
                                      self.head_dim, self.scale, self.window)
        return k.linear(mixed, self.w_o, self.b_o, residual=residual)


register_part("mixer", "gqa_attention", GQAAttention)
