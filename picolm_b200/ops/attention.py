"""Attention over the paged cache: the CUDA-core kernel, the mma.sync kernels (prefill, decode), the
tcgen05 prefill kernel, and the dispatcher `attention`."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc.build import attention_variant
from ._lib import (PAGE_TOKENS, SM_COUNT, KernelError, _check, _dev, _dt, _fn, _i32, _p, _stream, set_bounds,
                   status_word)


def attention_rows(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor,
                   tok_seq: torch.Tensor, block_table: torch.Tensor, num_kv_heads: int, scale: float,
                   window: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of q [T, H, hd] over the paged cache; returns [T, H*hd]."""
    _dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache")
    _i32(tok_pos, "tok_pos"), _i32(tok_seq, "tok_seq"), _i32(block_table, "block_table")
    T, H, hd = q.shape
    G = num_kv_heads
    if k_cache.dtype != q.dtype or k_cache.shape[1:] != (G, PAGE_TOKENS, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention: the cache must be [pages, {G}, {PAGE_TOKENS}, {hd}] of {q.dtype}")
    if hd > 256:
        raise KernelError(f"attention: head_dim {hd} exceeds 256, the largest this kernel takes")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    _cache_bounds("attention_simt", (), k_cache, block_table)
    _check(_fn("attention_simt", "plm_attention_rows")(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _dt(q, "q"), _p(tok_pos), _p(tok_seq), _p(block_table),
        block_table.shape[1], T, H, G, hd, float(scale), int(window or 0), _stream()), f"attention_rows T={T} H={H} hd={hd}")
    return out


def _cache_bounds(library, flags, k_cache, block_table) -> None:
    """The checked build's bounds for a kernel that walks `block_table` into `k_cache`."""
    set_bounds(library, flags, n_pages=k_cache.shape[0], n_seqs=block_table.shape[0],
               n_positions=block_table.shape[1] * PAGE_TOKENS, device=k_cache.device)


def attention_mma_supported(q: torch.Tensor) -> bool:
    """The tensor-core attention takes bfloat16 and head sizes that are multiples of 16 up to 256."""
    hd = q.shape[-1]
    return q.dtype == torch.bfloat16 and hd % 16 == 0 and 16 <= hd <= 256


def _attn_check(q, k_cache, v_cache, num_kv_heads):
    _dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache")
    T, H, hd = q.shape
    if not attention_mma_supported(q):
        raise KernelError(f"attention: {q.dtype} with head_dim {hd} is not supported by the tensor-core kernel "
                          f"(bfloat16, head_dim a multiple of 16 up to 256)")
    if k_cache.dtype != q.dtype or k_cache.shape[1:] != (num_kv_heads, PAGE_TOKENS, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention: the cache must be [pages, {num_kv_heads}, {PAGE_TOKENS}, {hd}] of {q.dtype}")
    if H % num_kv_heads:
        raise KernelError("attention: the number of heads is not a multiple of the number of KV heads")
    return T, H, hd


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_start: torch.Tensor,
                      seq_kv_len: torch.Tensor, block_table: torch.Tensor, max_new: int, num_kv_heads: int,
                      scale: float, window: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of every sequence's new tokens (rows seq_start[b]..seq_start[b+1] of q [T, H, hd])
    over its keys 0..seq_kv_len[b]-1 in the paged cache; returns [T, H*hd]."""
    T, H, hd = _attn_check(q, k_cache, v_cache, num_kv_heads)
    _i32(seq_start, "seq_start"), _i32(seq_kv_len, "seq_kv_len"), _i32(block_table, "block_table")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    lib, flags = attention_variant(hd)
    _cache_bounds(lib, flags, k_cache, block_table)
    _check(_fn(lib, "plm_attn_prefill", flags)(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(seq_start), _p(seq_kv_len), _p(block_table),
        block_table.shape[1], seq_kv_len.numel(), int(max_new), H, num_kv_heads, float(scale), int(window or 0),
        _stream()), f"attention_prefill(mma) T={T} H={H} hd={hd}", flops=2 * H * hd * T * int(max_new))
    return out


def attention_tc_supported(q: torch.Tensor) -> bool:
    """The tcgen05 prefill attention takes bfloat16 and head sizes 64 and 128."""
    return q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_start: torch.Tensor,
                         seq_kv_len: torch.Tensor, block_table: torch.Tensor, max_new: int, num_kv_heads: int,
                         scale: float, window: Optional[int] = None,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`attention_prefill` on the tcgen05 tensor cores (scores and the page's output in tensor memory,
    operands by TMA): same arguments, same result up to rounding; head sizes 64 and 128."""
    T, H, hd = _attn_check(q, k_cache, v_cache, num_kv_heads)
    if not attention_tc_supported(q):
        raise KernelError(f"attention_prefill_tc: head_dim {hd} of {q.dtype} is not supported (bfloat16, 64 or 128)")
    _i32(seq_start, "seq_start"), _i32(seq_kv_len, "seq_kv_len"), _i32(block_table, "block_table")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    lib, flags = attention_variant(hd, "attention_tc")
    _cache_bounds(lib, flags, k_cache, block_table)
    _check(_fn(lib, "plm_attn_tc_prefill", flags)(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(seq_start), _p(seq_kv_len), _p(block_table),
        block_table.shape[1], k_cache.shape[0], T, seq_kv_len.numel(), int(max_new), H, num_kv_heads, float(scale),
        int(window or 0), _p(status_word(q.device)), _stream()), f"attention_prefill_tc T={T} H={H} hd={hd}",
        flops=2 * H * hd * T * int(max_new))
    return out


DECODE_CLUSTER_SPLITS = 8       # up to this many ranges merge inside a thread-block cluster, without scratch


def decode_ctas_per_sm(head_dim: int, heads_per_kv_head: int) -> int:
    """How many CTAs of the decode kernel share an SM: its shared memory (three stages of a key and a value
    tile of 64 padded rows, and 9 or 16 query rows; csrc/attention_mma.cu) against the SM's 227 KB."""
    row = (head_dim + 8) * 2
    q_rows = (9 if heads_per_kv_head <= 8 else 16) * row
    if head_dim % 64 == 0:                                       # pages by TMA: unpadded tiles, 1024-byte aligned
        smem = q_rows + 1024 + 6 * 64 * head_dim * 2 + 64
    else:
        smem = q_rows + 6 * 64 * row
    return max(1, min(6, (227 * 1024) // (smem + 1024)))         # (registers allow six)


def decode_splits(n_tokens: int, num_heads: int, num_kv_heads: int, max_kv_len: int, head_dim: int = 64) -> int:
    """Into how many ranges the decode kernel cuts each sequence's keys.  Short contexts, where the whole
    grid runs at once (up to three CTAs an SM): as many ranges as that allows, up to the eight that merge
    inside a cluster, each of at least two and at most sixteen pages.  Longer contexts: as many ranges as
    make one wave of CTAs at full occupancy, each of at least eight pages (few long ranges read at 0.9 of the
    copy bandwidth where many short ones reach 0.7: every range pays for its start and its partial result);
    grids that fill the SMs without cutting get ranges of up to 64 pages (measured at batch 1, 8, 16 and 64 with
    2,048 to 32,768 keys)."""
    row_groups = (num_heads // num_kv_heads + 15) // 16
    ctas = max(1, n_tokens * num_kv_heads * row_groups)
    pages = max(1, (max_kv_len + PAGE_TOKENS - 1) // PAGE_TOKENS)
    per_sm = decode_ctas_per_sm(head_dim, num_heads // num_kv_heads)
    # (at most three CTAs an SM are counted on for the cluster form: a grid that fills the SMs to the brim keeps
    # the next kernel's CTAs, which would already be asking for their weights, off them; measured at batch 8)
    wave = min(3, per_sm) * SM_COUNT
    in_cluster = min(DECODE_CLUSTER_SPLITS, wave // ctas, max(1, pages // 2))
    if in_cluster >= 2 and pages <= (16 if ctas * in_cluster >= SM_COUNT else 8) * in_cluster:
        return in_cluster
    in_wave = per_sm * SM_COUNT // ctas
    if in_wave >= 2:
        return max(1, min(pages, in_wave, max(2, pages // 8)))
    return max(1, (pages + 63) // 64)


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor,
                     tok_seq: torch.Tensor, block_table: torch.Tensor, num_kv_heads: int, scale: float,
                     n_splits: int, window: Optional[int] = None, out: Optional[torch.Tensor] = None,
                     scratch: Optional[bool] = None) -> torch.Tensor:
    """Attention of single query tokens (one per row of q [T, H, hd], at position tok_pos[t] of sequence
    tok_seq[t]) over the paged cache, the keys of each cut into `n_splits` ranges.  Up to eight ranges are the
    CTAs of a thread-block cluster and merge through its shared memory; more ranges, or more CTAs than
    run at once, pass their partial results through a scratch buffer and a second kernel (`scratch` forces
    one way or the other).  Returns [T, H*hd]."""
    T, H, hd = _attn_check(q, k_cache, v_cache, num_kv_heads)
    _i32(tok_pos, "tok_pos"), _i32(tok_seq, "tok_seq"), _i32(block_table, "block_table")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    # Clusters are scheduled as a whole: past one wave of CTAs that costs more than the second kernel saves.
    ctas = T * num_kv_heads * ((H // num_kv_heads + 15) // 16) * n_splits
    if scratch is None:
        scratch = ctas > min(3, decode_ctas_per_sm(hd, H // num_kv_heads)) * SM_COUNT
    scratch = n_splits > 1 and (scratch or n_splits > DECODE_CLUSTER_SPLITS)
    ws = torch.empty((T * H * n_splits * (hd + 2),), dtype=torch.float32, device=q.device) if scratch else None
    lib, flags = attention_variant(hd)
    _cache_bounds(lib, flags, k_cache, block_table)
    _check(_fn(lib, "plm_attn_decode", flags)(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(ws), _p(tok_pos), _p(tok_seq), _p(block_table),
        block_table.shape[1], T, H, num_kv_heads, float(scale), int(window or 0), int(n_splits), k_cache.shape[0],
        _p(status_word(q.device)), _stream()),
        f"attention_decode T={T} H={H} hd={hd} splits={n_splits}", kernels=2 if scratch else 1)
    return out


class Rotation:
    """A rotary encoding as the kernels take it: cos / sin tables [positions, rotary_dim / 2] in float32,
    how many leading components of a head are rotated, and how they pair up ("half" or "adjacent")."""
    __slots__ = ("cos", "sin", "rotary_dim", "pairing")

    def __init__(self, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int, pairing: str):
        self.cos, self.sin, self.rotary_dim, self.pairing = cos, sin, rotary_dim, pairing


def attention_decode_rope_supported(qkv: torch.Tensor, kv, rotation: Optional[Rotation], head_dim: int) -> bool:
    """Whether the decode kernel can do this rotation and the cache write itself: bfloat16, a head size it
    takes, the whole head rotated in half-split pairs, a cache that this layer writes."""
    return (rotation is not None and qkv.dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and rotation.rotary_dim == head_dim and rotation.pairing == "half" and kv.writable
            and kv.k.dtype == torch.bfloat16 and rotation.cos is not None)


def attention_decode_rope(qkv: torch.Tensor, kv, step, num_heads: int, num_kv_heads: int, head_dim: int,
                          scale: float, rotation: Rotation, scratch: Optional[bool] = None) -> torch.Tensor:
    """A decode step's attention with the rotary encoding and the cache write folded in: `qkv`
    [T, (H + 2G) * hd] is the output of the QKV projection; queries and the new keys are rotated inside
    the kernel, the new keys and values are written to the cache at the tokens' positions, and the
    queries attend to everything up to and including them.  Returns [T, H * hd]."""
    _dev(qkv, "qkv"), _dev(kv.k, "k_cache"), _dev(kv.v, "v_cache")
    T = qkv.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if not attention_decode_rope_supported(qkv, kv, rotation, hd):
        raise KernelError("attention_decode_rope: not a case the fused kernel takes")
    if qkv.shape[1] != (H + 2 * G) * hd or kv.k.shape[1:] != (G, PAGE_TOKENS, hd) or kv.v.shape != kv.k.shape:
        raise KernelError("attention_decode_rope: qkv or the cache does not have the shape the heads imply")
    if step.max_position >= rotation.cos.shape[0]:
        raise KernelError(f"position {step.max_position} lies beyond the rotary table")
    n_splits = decode_splits(T, H, G, step.max_position + 1, hd)
    ctas = T * G * ((H // G + 15) // 16) * n_splits
    if scratch is None:
        scratch = ctas > min(3, decode_ctas_per_sm(hd, H // G)) * SM_COUNT
    scratch = n_splits > 1 and (scratch or n_splits > DECODE_CLUSTER_SPLITS)
    out = torch.empty((T, H * hd), dtype=qkv.dtype, device=qkv.device)
    ws = torch.empty((T * H * n_splits * (hd + 2),), dtype=torch.float32, device=qkv.device) if scratch else None
    lib, flags = attention_variant(hd)
    _cache_bounds(lib, flags, kv.k, kv.block_table)
    _check(_fn(lib, "plm_attn_decode_rope", flags)(
        _p(qkv), _p(kv.k), _p(kv.v), _p(out), _p(ws), _p(rotation.cos), _p(rotation.sin), _p(step.tok_pos),
        _p(step.tok_seq), _p(kv.block_table), kv.block_table.shape[1], T, H, G, float(scale), int(kv.window or 0),
        int(n_splits), kv.k.shape[0], _p(status_word(qkv.device)), _stream()), f"attention_decode_rope T={T} H={H} hd={hd} splits={n_splits}", kernels=2 if scratch else 1,
        nbytes=T * (step.max_position + 1) * 2 * G * hd * 2)
    return out


def attention(q: torch.Tensor, kv, step, num_kv_heads: int, scale: float) -> torch.Tensor:
    """Causal attention of the step's queries over their sequences' cached keys
    and values (`kv` is a `KVLayerCache`)."""
    if attention_mma_supported(q):
        if step.is_decode:
            splits = decode_splits(q.shape[0], q.shape[1], num_kv_heads, step.max_position + 1, q.shape[2])
            return attention_decode(q, kv.k, kv.v, step.tok_pos, step.tok_seq, kv.block_table, num_kv_heads, scale,
                                    splits, window=kv.window)
        prefill = attention_prefill_tc if attention_tc_supported(q) else attention_prefill
        return prefill(q, kv.k, kv.v, step.seq_start, step.seq_kv_len, kv.block_table, step.max_new,
                       num_kv_heads, scale, window=kv.window)
    return attention_rows(q, kv.k, kv.v, step.tok_pos, step.tok_seq, kv.block_table, num_kv_heads, scale,
                          window=kv.window)
