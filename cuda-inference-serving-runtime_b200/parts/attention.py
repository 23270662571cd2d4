"""Grouped-query attention over the paged cache.

Parity: runtime/model.py:110-115 (q, k, v projections without bias, rotation of q
and k, keys cached rotated, attention, output projection), runtime/reference.py:18-27
(consecutive query heads share a key/value head; scores scaled by 1/sqrt(D); causal
by construction).  q_proj, k_proj and v_proj are stacked into one matrix at load.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from ..config.spec import CacheUse
from ..ops import kernels
from .base import MIXERS, POSITIONS, Mixer, TensorNeed, build_part, register
from .linear import stream_target, as_tensor, linear, linear_to_stream, norm_fusable


# Keys per range of the split decode attention.  Ranges are [i * DECODE_RANGE, (i + 1) * DECODE_RANGE) in absolute
# positions whatever else is in the step, so the order in which a request's keys are summed depends on its own length
# alone: 256 keys are one tile for each of a CTA's four warps at head size 64, two at head size 128.  A large batch
# would rather have fewer, longer ranges (at 64 requests of 4096 tokens the step is a twentieth slower for it); that is
# the price of a sum that does not change with the neighbours.
DECODE_RANGE = 256
CLUSTER_MAX = 16           # key ranges of one request and head that one thread-block cluster can merge


@register(MIXERS, "gqa_attention")
class GQAAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, position (PartSpec), window (None or int), scale."""

    graph_safe = True
    accepts_pending_norm = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.hq = int(spec["num_heads"])
        self.hkv = int(spec["num_kv_heads"])
        self.dim = int(spec["head_dim"])
        self.window = spec.get("window")
        self.scale = float(spec.get("scale", self.dim ** -0.5))
        if self.hq % self.hkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.dim % 16 or not 16 <= self.dim <= 256:
            raise ValueError(f"head_dim {self.dim} is not supported: the attention kernels take multiples of 16 "
                             "from 16 to 256")
        self.position = build_part(POSITIONS, spec["position"], dtype, "position encoding")
        self.qkv = None
        self.o = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {"q_proj.weight": TensorNeed((self.hq * self.dim, self.hidden)),
                "k_proj.weight": TensorNeed((self.hkv * self.dim, self.hidden)),
                "v_proj.weight": TensorNeed((self.hkv * self.dim, self.hidden)),
                "o_proj.weight": TensorNeed((self.hidden, self.hq * self.dim))}

    def load(self, tensors):
        self.qkv = torch.cat((tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]), dim=0).contiguous()
        self.o = tensors["o_proj.weight"].contiguous()

    def kernel_jobs(self):
        return ([("elementwise.cu", {}, ()), kernels.attention_jobs(self.dim, self.dtype)]
                + kernels.attention_tcgen05_jobs(self.dim, self.dtype) + kernels.gemm_jobs(self.dtype) + self.position.kernel_jobs()
                + (kernels.skinny_jobs() + kernels.merge_proj_jobs() if self.dtype == torch.bfloat16 else []))

    def cache_use(self) -> CacheUse:
        return CacheUse("pages", kv_heads=self.hkv, head_dim=self.dim, window=self.window)

    # ---------------------------------------------------------------- the launch plan of a step
    def plan_key(self):
        return ("gqa_attention", kernels.PREFILL_TILE, kernels.WIDE_TILE, DECODE_RANGE)

    def step_plan(self, host):
        """Which CTAs the attention kernels launch for a step: portions of more than one token are cut into query
        tiles (request, first query), once per tile size of the two prompt kernels, a portion's last tile first (it
        has the longest key loop); single tokens are listed for the split kernel, whose number of key ranges comes
        from the longest context among them (or from the bound a captured graph was made for)."""
        from ..engine.batch import StepPlan

        tile_req, tile_q0, wide_req, wide_q0, dec_req = [], [], [], [], []
        longest = 0
        for r, n in enumerate(host.q_len):
            if n == 1:
                dec_req.append(r)
                longest = max(longest, host.ctx_len[r])
            else:
                for q0 in reversed(range(0, n, kernels.PREFILL_TILE)):
                    tile_req.append(r)
                    tile_q0.append(q0)
                for q0 in reversed(range(0, n, kernels.WIDE_TILE)):
                    wide_req.append(r)
                    wide_q0.append(q0)
        if dec_req and host.ctx_bound:
            longest = max(longest, host.ctx_bound)
        as_i32 = lambda values: np.asarray(values, dtype=np.int32)
        return StepPlan(
            arrays={"tile_req": as_i32(tile_req), "tile_q0": as_i32(tile_q0), "wide_req": as_i32(wide_req),
                    "wide_q0": as_i32(wide_q0), "dec_req": as_i32(dec_req)},
            info={"n_tiles": len(tile_req), "n_wide": len(wide_req), "n_decode": len(dec_req),
                  "n_splits": decode_ranges(longest)})

    def begin_step(self, ctx) -> None:
        self.position.rotation(ctx)          # the rotation tables of the step, shared by every layer with the same encoding

    def forward(self, h, ctx, cache):
        h0 = h                    # as it came: the pending norm, through which the output may go straight into the stream
        tokens = ctx.n_tokens
        hq, hkv, dim = self.hq, self.hkv, self.dim
        device = ctx.device
        rot = self.position.rotation(ctx)
        q = torch.empty((tokens, hq, dim), dtype=self.dtype, device=device)
        if cache.write and kernels.skinny_ok(tokens, self.qkv):
            # few tokens: one launch computes (the norm,) the projection, the rotation and the cache write
            rope = dict(cos=rot.cos if rot else None, sin=rot.sin if rot else None, rot_half=rot.rot_half if rot else 0,
                        interleaved=rot.interleaved if rot else False, q_out=q, k_cache=cache.k, v_cache=cache.v,
                        positions=ctx.positions, token_req=ctx.token_req, req_slot=ctx.req_slot,
                        block_table=cache.block_table, page_size=cache.page_size, hq=hq, hkv=hkv, dim=dim)
            if norm_fusable(h, tokens, self.qkv):
                x_out = h.new_stream_buffer()
                kernels.skinny_gemm(self.qkv, tokens, x=h.x, delta=h.delta, norm_w=h.weight, eps=h.eps, x_out=x_out,
                                    epilogue=kernels.EPI_ROPE, rope=rope)
                h.done(x_out)
            else:
                kernels.skinny_gemm(self.qkv, tokens, act=as_tensor(h), epilogue=kernels.EPI_ROPE, rope=rope)
        elif (cache.write and rot is not None and kernels.tcgen05_rope_ok(dim, rot.rot_half, rot.interleaved)
              and kernels.tcgen05_ok(as_tensor(h) if isinstance(h, torch.Tensor) else h.materialize_once(), self.qkv, fused=True)):
            # many tokens: rotation and cache write are the epilogue of the tcgen05 product
            kernels.gemm_tcgen05_rope(h if isinstance(h, torch.Tensor) else h.materialize_once(), self.qkv, dict(
                cos=rot.cos, sin=rot.sin, q_out=q, k_cache=cache.k, v_cache=cache.v, positions=ctx.positions,
                token_req=ctx.token_req, req_slot=ctx.req_slot, block_table=cache.block_table, page_size=cache.page_size,
                hq=hq, hkv=hkv, dim=dim))
        else:
            h = h if isinstance(h, torch.Tensor) else h.materialize_once()
            if cache.write:
                proj = linear(h, self.qkv)
                k_col, v_col = hq * dim, (hq + hkv) * dim
            else:  # this run entry reads another entry's keys and values: queries only
                proj = linear(h, self.qkv[: hq * dim])
                k_col = v_col = -1
            kernels.rope_store(proj, k_col, v_col, rot.cos if rot else None, rot.sin if rot else None,
                               rot.rot_half if rot else 0, rot.interleaved if rot else False, q,
                               cache.k if cache.write else None, cache.v if cache.write else None,
                               ctx.token_req, ctx.positions, ctx.req_slot, cache.block_table, cache.page_size, hq, hkv, dim)
        out = torch.empty((tokens, hq, dim), dtype=self.dtype, device=device)
        plan = ctx.plan_for(self)
        if plan.info["n_tiles"] and kernels.attn_prefill_wide_ok(q, cache.k, cache.page_size):
            kernels.attn_prefill_wide(q, out, cache.k, cache.v, ctx.req_slot, cache.block_table, plan["wide_req"], plan["wide_q0"],
                                      ctx.q_start, ctx.q_len, ctx.ctx_len, hq, hkv, cache.page_size, self.scale, self.window)
        elif plan.info["n_tiles"]:
            kernels.attn_prefill(q, out, cache.k, cache.v, ctx.req_slot, cache.block_table, plan["tile_req"], plan["tile_q0"],
                                 ctx.q_start, ctx.q_len, ctx.ctx_len, hq, hkv, cache.page_size, self.scale, self.window)
        n_decode = plan.info["n_decode"]
        if n_decode:
            n_splits = plan.info["n_splits"]
            partial = torch.empty((n_decode, hq, n_splits, dim), dtype=torch.float32, device=device)
            stats = torch.empty((n_decode, hq, n_splits, 2), dtype=torch.float32, device=device)
            # a step of single tokens only, with a small output projection: the merge of the key ranges is the prologue
            # of that projection (one launch of a thread-block cluster instead of the merge kernel and the product)
            fused = (n_decode == tokens and self.dtype == torch.bfloat16 and dim <= kernels.TENSOR_CORE_MAX_HEAD_DIM
                     and kernels.merge_out_proj_ok(n_decode, hq, dim, self.o))
            kernels.attn_decode(q, out, cache.k, cache.v, ctx.req_slot, cache.block_table, plan["dec_req"], n_decode, ctx.q_start,
                                ctx.ctx_len, partial, stats, hq, hkv, cache.page_size, self.scale, self.window,
                                DECODE_RANGE, n_splits, merge=not fused)
            if fused:
                x = stream_target(h0, tokens, self.hidden)
                if x is not None:     # straight into the residual stream
                    kernels.merge_out_proj(partial, stats, n_splits, plan["dec_req"], ctx.q_start, n_decode, hq, dim, self.o, x,
                                           accumulate=True)
                    return None
                projected = torch.empty((tokens, self.hidden), dtype=torch.float32, device=device)
                return kernels.merge_out_proj(partial, stats, n_splits, plan["dec_req"], ctx.q_start, n_decode, hq, dim, self.o, projected)
        return linear_to_stream(out.view(tokens, hq * dim), self.o, h0)


def decode_ranges(longest_context: int) -> int:
    """How many key ranges of DECODE_RANGE the split kernel is launched with, per request and key head, for contexts
    up to `longest_context`.  Ranges beyond a request's own length are empty and change nothing in its sum, so the
    count may be any bound; beyond CLUSTER_MAX it is rounded up to whole clusters for the cluster merge."""
    n = max(1, -(-longest_context // DECODE_RANGE))
    if n > CLUSTER_MAX:
        n = -(-n // CLUSTER_MAX) * CLUSTER_MAX
    return n
