"""Latent attention: a token keeps one latent vector and one rotated key part for all heads.

``q = W_q h`` per head ``[D plain | R rotated]``; ``W_dkv h`` gives ``C + R`` channels: the first
``C``, RMS-normed with a plain weight, are the latent vector ``c``, the last ``R`` one rotated key
part shared by the heads.  A head's key is ``[W_uk c | rotated part]``, its value ``W_uv c``, the
score ``(q_plain . k_plain + q_rot . k_rot) * scale`` under a sliding window, softmax, and ``W_o``
on the joined heads.  Rotation: of the first ``rotary_dims`` channels of the rotated part, channel
``2i`` with ``2i + 1`` by the angle ``p * base^(-2i / rotary_dims)``.

Options: ``q_rank`` > 0 sends the queries through a latent of their own, ``c_q = RMSnorm(W_dq h)``
(weight ``dq.norm``), ``q = W_uq c_q``; ``rope_dim = 0`` leaves the rotated part out altogether
(no positions); ``head_gate`` multiplies head ``n``'s output by ``sigmoid(W_g h)_n``;
``own_latent = False`` makes a layer without a down-projection of its own: it reads the latent
vectors that ANOTHER layer of the same ``kv_rank`` cached (the plan gives it that layer's cache to
read), with its own up-projections, queries and everything else.

Only ``c`` and the rotated part are cached (two planes of a paged cache; one without it).  The key up-projection
is folded into the query (``q_lat = W_uk^T q_plain``, a batched product over heads), the kernel
attends over ``[c | r]`` with values ``c``, and the value up-projection (a second batched product)
follows: keys and values of the heads are never formed.

Long portions of a design without a rotated part (bfloat16, head sizes up to 128) take the other
order: the step's requests' cached latent vectors are gathered, ``k = W_uk c`` and ``v = W_uv c``
are formed for them by two products into a scratch cache of the step, and the grouped-query
attention kernels (tcgen05 for prompts) run over that.  Heads narrower than the kernels' 64 or 128
channels are padded with zero rows of the up-projections (and zero columns of ``W_o``), so nothing
is copied.  The cache still holds ``c`` alone.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops import latent, prenorm
from .base import Mixer, PagedKVSpec, TensorSpec, register_mixer


class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, nope_dim: int, rope_dim: int, v_dim: int,
                 kv_rank: int, scale: float, window: int = 0, rotary_dims: int | None = None,
                 rotary_base: float = 10000.0, latent_eps: float = 1e-6, prefix: str = "mix",
                 q_rank: int = 0, head_gate: bool = False, own_latent: bool = True):
        self.hidden_size, self.H = int(hidden_size), int(num_heads)
        self.D, self.R, self.Vd, self.C = int(nope_dim), int(rope_dim), int(v_dim), int(kv_rank)
        self.scale, self.window = float(scale), int(window)
        self.rot = int(self.R if rotary_dims is None else rotary_dims)
        if self.rot % 2 or self.rot > self.R:
            raise ValueError(f"{self.rot} rotated channels of {self.R}: must be even and fit")
        self.base, self.eps = float(rotary_base), float(latent_eps)
        self.prefix = prefix + "." if prefix else ""
        self.Q, self.gated, self.own = int(q_rank), bool(head_gate), bool(own_latent)
        if not self.own and self.R:
            raise ValueError("a layer that reads another layer's latent vectors has no rotated "
                             "key part of its own")
        # the plain form: queries straight from h, a rotated part, no gate (one fused kernel)
        self.classic = self.Q == 0 and self.R > 0 and not self.gated and self.own

    def _n(self, name):
        return self.prefix + name

    def tensor_specs(self):
        H, D, R, Vd, C, W = self.H, self.D, self.R, self.Vd, self.C, self.hidden_size
        out = []
        if self.Q:
            out += [TensorSpec(self._n("dq"), (self.Q, W)),
                    TensorSpec(self._n("dq.norm"), (self.Q,), "f32"),
                    TensorSpec(self._n("uq"), (H * (D + R), self.Q))]
        else:
            out.append(TensorSpec(self._n("q"), (H * (D + R), W)))
        if self.own:
            out += [TensorSpec(self._n("dkv"), (C + R, W)),
                    TensorSpec(self._n("dkv.norm"), (C,), "f32")]
        if self.gated:
            out.append(TensorSpec(self._n("g"), (H, W)))
        return out + [TensorSpec(self._n("uk"), (H * D, C)),
                      TensorSpec(self._n("uv"), (H * Vd, C)),
                      TensorSpec(self._n("o"), (W, H * Vd))]

    def load(self, tensors, dtype, device):
        H, D, Vd, C = self.H, self.D, self.Vd, self.C
        # one product for everything that reads h: (q or dq) | (dkv) | (g), padded to 8 rows
        rows = [tensors[self._n("dq" if self.Q else "q")]]
        self.c_col = rows[0].shape[0]
        if self.own:
            rows.append(tensors[self._n("dkv")])
        self.g_col = sum(r.shape[0] for r in rows)
        if self.gated:
            rows.append(tensors[self._n("g")])
        n = sum(r.shape[0] for r in rows)
        if -n % 8 and not self.classic:
            rows.append(torch.zeros((-n % 8, self.hidden_size), dtype=rows[0].dtype, device=device))
        self.q_dkv = ops.Linear(torch.cat(rows, dim=0) if len(rows) > 1 else rows[0])
        self.latent_w = tensors[self._n("dkv.norm")].float().contiguous() if self.own else None
        self.q_w = tensors[self._n("dq.norm")].float().contiguous() if self.Q else None
        self.uq = ops.Linear(tensors[self._n("uq")]) if self.Q else None
        self.uk = tensors[self._n("uk")].view(H, D, C)                     # q_lat = q_plain @ uk[h]
        self.uv_t = tensors[self._n("uv")].view(H, Vd, C).transpose(1, 2)  # values = o_lat @ uv[h]^T
        self.out = ops.Linear(tensors[self._n("o")], None, out_dtype=torch.float32)
        i = np.arange(self.rot // 2, dtype=np.float64)
        freq = np.power(np.float64(self.base), -2.0 * i / self.rot).astype(np.float32)
        self.freq = torch.from_numpy(freq).to(device)
        # keys and values formed for long portions: up-projections padded to the kernels' head size
        self.HDp = 0
        widest = max(D, Vd)
        if (self.R == 0 and self.Q and not self.classic and self.uk.dtype == torch.bfloat16
                and widest <= 128):
            P = self.HDp = 64 if widest <= 64 else 128

            def rows(w, n):          # [H * n, in] -> [H * P, in], zero rows behind each head's n
                if n == P:
                    return w
                out = torch.zeros((H, P, w.shape[1]), dtype=w.dtype, device=w.device)
                out[:, :n] = w.view(H, n, w.shape[1])
                return out.view(H * P, w.shape[1])
            self.uq_wide = ops.Linear(rows(tensors[self._n("uq")], D))
            self.uk_wide = rows(tensors[self._n("uk")], D).contiguous()
            self.uv_wide = rows(tensors[self._n("uv")], Vd).contiguous()
            wo = tensors[self._n("o")]
            if Vd != P:
                wide = torch.zeros((wo.shape[0], H, P), dtype=wo.dtype, device=wo.device)
                wide[:, :, :Vd] = wo.view(wo.shape[0], H, Vd)
                wo = wide.view(wo.shape[0], H * P)
            self.out_wide = ops.Linear(wo, None, out_dtype=torch.float32)

    def cache_spec(self):
        if self.R == 0:
            return PagedKVSpec(1, self.C, self.window, planes=((1, self.C),))
        return PagedKVSpec(1, self.C, self.window, planes=((1, self.C), (1, self.R)))

    def forward(self, x, ctx, cache):
        H, D, R, C = self.H, self.D, self.R, self.C
        T = x.shape[0]
        qd = self.q_dkv(x)                        # [T, (H (D + R) or Q) | (C + R) | (H) | pad]
        if self.classic:
            c_pages, r_pages = cache.pages
            q_rot = latent.prepare(qd[:, :H * (D + R) + C + R], H, D, R, C, self.rot, self.freq,
                                   self.latent_w, self.eps, ctx.positions,
                                   cache.slot_mapping if cache.write else None, c_pages, r_pages)
            q_all = qd
        else:
            if R:
                raise NotImplementedError("a rotated part together with a query latent or a gate")
            c_pages, r_pages, q_rot = cache.pages[0], None, None
            write = cache.write and self.own
            cq = latent.norms(qd, 0, self.Q, self.q_w, self.c_col, C, self.latent_w, self.eps,
                              cache.slot_mapping if write else None, c_pages)
            if self.HDp and x.dtype == torch.bfloat16 and ctx.max_q_len >= FORMED_MIN_QUERY_ROWS:
                o = self._over_formed_keys(cq, ctx, cache, c_pages)
                if o is not None:
                    if self.gated:
                        prenorm.head_gate(o, qd[:, self.g_col:self.g_col + H], H, self.HDp)
                    return self.out_wide(o)
            q_all = self.uq(cq) if self.Q else qd
        q_plain = q_all[:, :H * (D + R)].unflatten(1, (H, D + R))[:, :, :D].transpose(0, 1)
        q_lat = ops.bmm_f32_out(q_plain, self.uk)                 # [H, T, C] fp32
        o_lat = latent.attention(q_lat, q_rot, c_pages, r_pages, cache.block_table, ctx,
                                 cache.window, self.scale, cache.page_size)
        o = torch.bmm(o_lat, self.uv_t)                           # [H, T, Vd]
        o = o.transpose(0, 1).reshape(T, H * self.Vd)
        if self.gated:
            prenorm.head_gate(o, qd[:, self.g_col:self.g_col + H], H, self.Vd)
        return self.out(o)


    def _over_formed_keys(self, cq, ctx, cache, c_pages):
        """Attention of a step with long portions over keys and values formed from the cached
        latent vectors -> ``[T, H * HDp]``, or ``None`` where the scratch would be too large.
        Request ``b`` owns the pages ``b W .. (b + 1) W - 1`` of the scratch, ``W`` the pages the
        longest request of the step holds (under graph capture: the block table's width); what
        lies behind a request's last token is formed from whatever the table names there and is
        never seen."""
        from ..ops import attention_bf16
        H, P, C = self.H, self.HDp, self.C
        page, table = cache.page_size, cache.block_table
        B = ctx.num_seqs
        if ctx.capturing or not ctx.q_lens_host:
            W = table.shape[1]
        else:
            longest = max(a + n for a, n in zip(ctx.q_starts_host, ctx.q_lens_host))
            W = min(table.shape[1], -(-longest // page))
        rows = B * W * page
        if rows > FORMED_MAX_ROWS or not attention_bf16.supports(P, H, H):
            return None
        c, own = latent.gather_pages(c_pages, table, B, W)                  # [rows, C], [B, W]
        kv = torch.empty((2, B * W, page, H, P), dtype=c.dtype, device=c.device)
        torch.mm(c, self.uk_wide.t(), out=kv[0].view(rows, H * P))
        torch.mm(c, self.uv_wide.t(), out=kv[1].view(rows, H * P))
        q = self.uq_wide(cq)
        return attention_bf16.try_run(q, kv, own, ctx, H, H, P, self.scale, cache.window, page)


# Portions of at least this many rows take the formed keys (the tcgen05 prompt kernel's tile),
# and a step's scratch holds at most this many tokens' keys and values.
FORMED_MIN_QUERY_ROWS = 64
FORMED_MAX_ROWS = 1 << 17


register_mixer("latent_attention", LatentAttention)
