"""Attention over one latent vector a position.

    q      = Wq x                       (or  Wuq . rmsnorm(Wdq x)  when the queries pass a latent of their own)
    c, kr  = split(Wdkv x);  c <- rmsnorm(c);  kr <- rotate(kr)          cached: [c | kr], one row a position
    head h:  score(i, j) = scale * ( q_plain[i, h] . (Wuk_h c_j)  +  rotate(q_rot[i, h]) . kr_j )
             out[i, h]   = Wuv_h . sum_j softmax_j(score) c_j
    y      = Wo . (concat(heads) * sigmoid(Wg x))                        (the gate only if the mixer has one)

The read-out matrices never touch the cache: the plain query part is taken through Wuk_h first
(q'[i, h] = Wuk_h^T q_plain[i, h], as wide as the latent), so that a score is one dot product of rank + rot_dim
elements against a cached row, every head reads the same rows, and the attention's result stays in the latent
space until Wuv_h is applied to it.  Queries and results are laid out head by head ([head][token][..]) in
between, so that both per-head products are one grouped product with the heads as groups.

Rotation: neighbouring pairs (2i, 2i + 1) of the first ``rotary_dims`` elements of the rot_dim part, pair i at
base^(-2i / rotary_dims); angles, norms and scores are 32-bit.
"""
from __future__ import annotations

import torch

from ..cache.specs import CacheSpec, PagedSpec, PagedTensorSpec
from ..kernels import ops
from ..weights.loader import TensorDecl
from .attention import _common_dtype, general_attention
from .base import Mixer, build_part, register_part
from .specs import AdjacentRotarySpec


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        s = spec
        if s.rotary_dims % 2 or not 0 <= s.rotary_dims <= s.rot_dim:
            raise ValueError(f"rotary_dims={s.rotary_dims}: even and at most rot_dim={s.rot_dim}")
        if s.window is not None and s.window < 1:
            raise ValueError(f"window={s.window}: a window holds at least the query's own position")
        if s.kv_rank + s.rot_dim > ops.ATTENTION_MAX_KEY_DIM or s.kv_rank > ops.ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"kv_rank={s.kv_rank}, rot_dim={s.rot_dim}: a cached row holds at most "
                             f"{ops.ATTENTION_MAX_KEY_DIM} elements, a latent at most {ops.ATTENTION_MAX_VALUE_DIM}")
        self.q_width = s.n_heads * (s.head_dim + s.rot_dim)
        self.row = s.kv_rank + s.rot_dim
        self.o_size = s.n_heads * s.value_dim
        self.rotary = build_part(AdjacentRotarySpec(rotary_dim=max(2, s.rotary_dims), theta=s.rotary_base))
        self._groups = {}

    def cache_spec(self):
        return CacheSpec(paged=PagedSpec((PagedTensorSpec("kv", (self.row,), lead_dims=0),), self.spec.window))

    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        d = []
        if s.q_rank:
            d += [TensorDecl(p + "dq", (s.q_rank, s.hidden)), TensorDecl(p + "dq.norm", (s.q_rank,), init="ones"),
                  TensorDecl(p + "uq", (self.q_width, s.q_rank))]
        else:
            d.append(TensorDecl(p + "q", (self.q_width, s.hidden)))
        d += [TensorDecl(p + "dkv", (self.row, s.hidden)), TensorDecl(p + "dkv.norm", (s.kv_rank,), init="ones"),
              TensorDecl(p + "uk", (s.n_heads * s.head_dim, s.kv_rank)),
              TensorDecl(p + "uv", (s.n_heads * s.value_dim, s.kv_rank))]
        if s.output_gate:
            d.append(TensorDecl(p + "g", (self.o_size, s.hidden)))
        d.append(TensorDecl(p + "o", (s.hidden, self.o_size)))
        return d

    def load(self, src, rt):
        super().load(src, rt)
        s, p = self.spec, self.spec.prefix
        H, D, V, C = s.n_heads, s.head_dim, s.value_dim, s.kv_rank
        # one product for everything that reads the mixer's input: [q or dq | dkv | g]
        first = [src.get(p + ("dq" if s.q_rank else "q")), src.get(p + "dkv")]
        if s.output_gate:
            first.append(src.get(p + "g"))
        dt = _common_dtype(first)
        self.w_in = torch.cat([w.to(dt) for w in first], dim=0).contiguous()
        self.w_uq = src.get(p + "uq") if s.q_rank else None
        self.q_norm = src.get(p + "dq.norm") if s.q_rank else None
        self.c_norm = src.get(p + "dkv.norm")
        # groups = heads: [H, C, D] takes a head's plain query part into the latent space (Wuk_h transposed),
        # [H, V, C] takes a head's result out of it
        self.w_uk_t = src.get(p + "uk").view(H, D, C).transpose(1, 2).contiguous()
        self.w_uv = src.get(p + "uv").view(H, V, C).contiguous()
        self.w_o = src.get(p + "o")
        self.rotary.load(src, rt)

    def _head_groups(self, T: int):
        """Where each head's rows begin when rows lie head by head, and the list of heads (the grouped products'
        group offsets and active groups).  Made once per step size, outside graph captures."""
        g = self._groups.get(T)
        if g is None:
            H, dev = self.spec.n_heads, self.rt.device
            g = ((torch.arange(H + 1, dtype=torch.int32, device=dev) * T).to(torch.int32),
                 torch.cat([torch.arange(H, dtype=torch.int32, device=dev),
                            torch.full((1,), -1, dtype=torch.int32, device=dev)]))
            if not (dev.type == "cuda" and torch.cuda.is_current_stream_capturing()):
                self._groups[T] = g
        return g

    def forward_add(self, x, h, batch, cache):
        self.forward_into(x, h, batch, cache, accumulate=True)

    def forward_into(self, x, out, batch, cache, accumulate=False):
        s, rt, st = self.spec, self.rt, batch.stream
        T, H, D, R, V, C = x.shape[0], s.n_heads, s.head_dim, s.rot_dim, s.value_dim, s.kv_rank
        row = self.row
        proj = rt.empty(T, self.w_in.shape[0])
        ops.linear(x, self.w_in, proj, status=batch.status, stream=st, after_short_kernel=True)
        if s.q_rank:
            cq = rt.empty(T, s.q_rank)
            ops.rmsnorm_rows(proj[:, :s.q_rank], self.q_norm, s.norm_eps, cq, stream=st)
            q = rt.empty(T, self.q_width)
            ops.linear(cq, self.w_uq, q, status=batch.status, stream=st)
            rest = s.q_rank
        else:
            q = proj[:, :self.q_width]
            rest = self.q_width
        dkv = proj[:, rest:rest + row]
        gate = proj[:, rest + row:] if s.output_gate else None
        pages = cache.pages["kv"]
        q_plain = rt.empty(H, T, D)
        q_full = rt.empty(H, T, row)
        cos_sin = self.rotary.table(batch) if s.rotary_dims > 0 else None
        ops.latent_prep(q, dkv, batch.positions, batch.token_seq, batch.seq_slot, self.c_norm, s.norm_eps, cos_sin,
                        s.rotary_dims, q_plain, q_full, pages, cache.block_table, cache.page_size, H, D, R, C,
                        write_cache=cache.writes, status=batch.status, stream=st)
        offsets, heads = self._head_groups(T)
        ops.grouped_linear(q_plain.view(H * T, D), self.w_uk_t, q_full.view(H * T, row)[:, :C], offsets, heads, T,
                           status=batch.status, stream=st)
        o_lat = rt.empty(H, T, C)
        general_attention(q_full, row, T * row, pages, pages, row, row, o_lat, C, T * C, batch, cache, H, 1, row, C,
                          s.window, s.scale, None, rt)
        o_heads = rt.empty(H, T, V)
        ops.grouped_linear(o_lat.view(H * T, C), self.w_uv, o_heads.view(H * T, V), offsets, heads, T,
                           status=batch.status, stream=st)
        attn = rt.empty(T, self.o_size)
        ops.heads_to_tokens(o_heads, attn, gate=gate, stream=st)
        ops.linear(attn, self.w_o, out, accumulate=accumulate, status=batch.status, stream=st, after_short_kernel=True)


register_part("latent_attention", LatentAttention, replace=True)
