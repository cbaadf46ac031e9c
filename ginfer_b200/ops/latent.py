"""Latent attention over a paged cache of one latent vector and one rotated key part a token
(``csrc/latent_attention.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import _code, _cuda, _fn, _ok, _p, _stream


def prepare(qd: torch.Tensor, H: int, D: int, R: int, C: int, rot: int, freq: torch.Tensor,
            cnorm_w: torch.Tensor, eps: float, positions: torch.Tensor, slot_mapping,
            c_pages: torch.Tensor, r_pages: torch.Tensor) -> torch.Tensor:
    """``qd [T, H (D + R) + C + R]``: the heads' queries ``[D plain | R rotated]``, then the
    down-projection ``[C | R]``.  Writes the normed latent vector and the rotated key part into the
    token's cache slot (``slot_mapping``; ``None``: no write) and returns the heads' rotated query
    parts ``[T, H, R]`` in fp32."""
    _cuda(qd, freq, cnorm_w, positions, slot_mapping, c_pages, r_pages)
    T = qd.shape[0]
    assert qd.dim() == 2 and qd.stride(1) == 1 and qd.shape[1] == H * (D + R) + C + R
    assert freq.dtype == torch.float32 and freq.numel() == rot // 2
    assert cnorm_w.dtype == torch.float32 and cnorm_w.numel() == C
    assert c_pages.is_contiguous() and r_pages.is_contiguous() and c_pages.dtype == qd.dtype
    assert c_pages.shape[-1] == C and r_pages.shape[-1] == R
    q_rot = torch.empty((T, H, R), dtype=torch.float32, device=qd.device)
    f = _fn("latent_attention", "gf_latent_prepare",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _ok(f(_p(qd), qd.stride(0), H, D, R, C, rot, _p(freq), _p(cnorm_w), float(eps),
          _p(positions), _p(slot_mapping), _p(c_pages), _p(r_pages), _p(q_rot), T,
          _code(qd.dtype), _stream()), "latent_prepare")
    return q_rot


def norms(proj: torch.Tensor, q_col: int, Q: int, q_w, c_col: int, C: int, c_w, eps: float,
          slot_mapping, c_pages):
    """Out of a projection row ``proj [T, ...]``: the query latent (``Q`` channels from ``q_col``)
    RMS-normed with ``q_w`` and returned ``[T, Q]`` in the row's dtype (``None`` for ``Q == 0``),
    and the key/value latent (``C`` channels from ``c_col``) RMS-normed with ``c_w`` into the
    token's slot of ``c_pages`` (skipped without ``slot_mapping``)."""
    _cuda(proj, q_w, c_w, slot_mapping, c_pages)
    T = proj.shape[0]
    assert proj.dim() == 2 and proj.stride(1) == 1
    assert q_col + Q <= proj.shape[1] and (slot_mapping is None or c_col + C <= proj.shape[1])
    for w, n in ((q_w, Q), (c_w, C)):
        assert w is None or (w.dtype == torch.float32 and w.numel() == n and w.is_contiguous())
    if slot_mapping is not None:
        assert c_pages.is_contiguous() and c_pages.dtype == proj.dtype and c_pages.shape[-1] == C
    cq = torch.empty((T, Q), dtype=proj.dtype, device=proj.device) if Q else None
    f = _fn("latent_attention", "gf_latent_norms",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_float,
             c_void_p, c_void_p, c_int, c_int, c_void_p])
    _ok(f(_p(proj), proj.stride(0), int(q_col), int(Q), _p(q_w), _p(cq), int(c_col), int(C),
          _p(c_w), float(eps), _p(slot_mapping), _p(c_pages), T, _code(proj.dtype), _stream()),
        "latent_norms")
    return cq


def gather_pages(c_pages: torch.Tensor, block_table: torch.Tensor, B: int, W: int):
    """The latent vectors that the first ``W`` entries of the ``B`` requests' block tables name,
    side by side: ``(c [B * W * page, C], own [B, W])``, ``own`` the block table under which ``c``,
    seen as ``B * W`` pages, is a cache of its own (request ``b`` owns pages ``b W .. b W + W -
    1``).  Entries behind a request's last page are clamped to the pool and never read as keys."""
    _cuda(c_pages, block_table)
    assert c_pages.is_contiguous() and block_table.dtype == torch.int32
    assert block_table.stride(1) == 1 and B <= block_table.shape[0] and W <= block_table.shape[1]
    num_pages, page, C = c_pages.shape[0], c_pages.shape[1], c_pages.shape[-1]
    assert c_pages.numel() == num_pages * page * C
    c = torch.empty((B * W * page, C), dtype=c_pages.dtype, device=c_pages.device)
    own = torch.empty((B, W), dtype=torch.int32, device=c_pages.device)
    f = _fn("latent_attention", "gf_latent_gather",
            [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_void_p])
    rc = f(_p(c_pages), _p(block_table), block_table.stride(0), int(B), int(W), page, C,
           c_pages.element_size(), num_pages, _p(c), _p(own), _stream())
    if rc == -3:
        raise ValueError(f"gather of {B} x {W} pages of {page} x {C}")
    _ok(rc, "latent_gather")
    return c, own


KEY_TILE = 64           # keys a tile of the tensor-core kernel
MAX_SPLITS = 8
MIN_TILES_A_SPLIT = 4   # a share shorter than this costs more in the merge than it saves


def key_splits(num_tokens: int, num_heads: int, max_keys: int, sms: int = 148) -> int:
    """How many blocks share the keys of a token: one unless the step's blocks would leave most
    SMs idle and a token has several tiles of keys."""
    blocks = num_tokens * -(-num_heads // 16)
    tiles = -(-max(1, max_keys) // KEY_TILE)
    if blocks * 2 > sms or tiles < 2 * MIN_TILES_A_SPLIT:
        return 1
    return max(1, min(tiles // MIN_TILES_A_SPLIT, sms // blocks, MAX_SPLITS))


def attention(q_lat: torch.Tensor, q_rot: torch.Tensor, c_pages: torch.Tensor,
              r_pages: torch.Tensor, block_table: torch.Tensor, ctx, window: int, scale: float,
              page_size: int) -> torch.Tensor:
    """``q_lat [H, T, C]`` and ``q_rot [T, H, R]`` in fp32 against the cache; returns the
    softmax-weighted latent vectors ``[H, T, C]`` in the cache's dtype.  ``ctx.max_kv_len`` (if
    there) bounds the keys of a token and decides whether several blocks share them."""
    _cuda(q_lat, q_rot, c_pages, r_pages, block_table)
    H, T, C = q_lat.shape
    R = q_rot.shape[2] if q_rot is not None else 0       # no rotated part: both are None
    assert q_lat.dtype == torch.float32 and q_lat.is_contiguous()
    assert q_rot is None or (q_rot.dtype == torch.float32 and q_rot.is_contiguous()
                             and q_rot.shape[:2] == (T, H))
    assert (R == 0) == (r_pages is None)
    out = torch.empty((H, T, C), dtype=c_pages.dtype, device=q_lat.device)
    nsplit, part_o, part_ml = 1, None, None
    max_keys = int(getattr(ctx, "max_kv_len", 0) or 0)
    if c_pages.dtype == torch.bfloat16 and max_keys > 0:
        nsplit = key_splits(T, H, min(max_keys, window) if window > 0 else max_keys)
        if nsplit > 1:
            part_o = torch.empty((nsplit, T, H, C), dtype=torch.float32, device=q_lat.device)
            part_ml = torch.empty((nsplit, T, H, 2), dtype=torch.float32, device=q_lat.device)
    f = _fn("latent_attention", "gf_latent_attention",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
             c_void_p, c_void_p], kernels=2 if nsplit > 1 else 1)
    rc = f(_p(q_lat), _p(q_rot), _p(c_pages), _p(r_pages), _p(block_table),
           block_table.stride(0), _p(ctx.seq_of_token), _p(ctx.positions), _p(out), T, H, C, R,
           int(page_size), int(window), float(scale), _code(c_pages.dtype), nsplit, _p(part_o),
           _p(part_ml), _stream())
    if rc == -3:
        raise ValueError(f"latent attention takes latent vectors of up to 1024 channels whose key "
                         f"tile fits shared memory; got kv_rank={C}, rot_dim={R}")
    _ok(rc, "latent_attention")
    return out
