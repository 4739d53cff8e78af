"""Paged key / value cache for single-token decode with PoPE attention.

The reference has no cache: every decode step calls ``flash_attn_with_pope`` with the full K and V
(PoPE_pytorch/attention.py:75-145; the query then sits at the last position, PoPE_pytorch/pope.py:64).
This is the serving-side step either side of that call: ``append`` writes the new rows of k and v into
fixed-size pages, ``decode`` attends one new query row per (batch, head) over everything a sequence holds.
Raw k is cached; the polar transform is applied inside the decode kernel as the keys stream through
shared memory, so cached entries do not depend on the phase bias.

Page bookkeeping (free list, page table, lengths) is host policy and lives here; the library only reads the
table (``pope_b200_kv_append`` / ``pope_b200_attn_decode_paged`` in include/pope_b200.h).  All arithmetic is
in the CUDA library; there is no fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _native as N


class PageAllocator:
    """Host-side free list and page table of a pool of ``num_pages`` pages; no device memory.

    ``table[b]`` lists the physical pages of sequence ``b`` in logical order; ``lens[b]`` is its length in keys."""

    def __init__(self, batch: int, num_pages: int, page_size: int, max_pages_per_seq: int):
        if page_size <= 0 or page_size % 64 != 0:
            raise ValueError("page_size must be a positive multiple of 64")
        self.batch, self.num_pages, self.page_size, self.max_pages_per_seq = batch, num_pages, page_size, max_pages_per_seq
        self.free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() hands out page 0 first
        self.table: List[List[int]] = [[] for _ in range(batch)]
        self.lens: List[int] = [0] * batch

    def pages_needed(self, b: int, n_new: int) -> int:
        need = -(-(self.lens[b] + n_new) // self.page_size)
        return max(0, need - len(self.table[b]))

    def reserve(self, n_new: int, rows: Optional[Sequence[int]] = None) -> List[tuple]:
        """Map the pages that ``n_new`` more keys per sequence need; returns the new (b, logical, physical) entries.
        Raises (and changes nothing) when the pool or a sequence's table is too small."""
        rows = range(self.batch) if rows is None else rows
        want = [(b, self.pages_needed(b, n_new)) for b in rows]
        if sum(n for _, n in want) > len(self.free):
            raise RuntimeError("paged KV cache: out of pages")
        for b, n in want:
            if len(self.table[b]) + n > self.max_pages_per_seq:
                raise RuntimeError("paged KV cache: sequence longer than max_pages_per_seq * page_size")
        new = []
        for b, n in want:
            for _ in range(n):
                pg = self.free.pop()
                new.append((b, len(self.table[b]), pg))
                self.table[b].append(pg)
        return new

    def advance(self, n_new: int, rows: Optional[Sequence[int]] = None) -> None:
        for b in (range(self.batch) if rows is None else rows):
            self.lens[b] += n_new

    def release(self, b: int) -> None:
        """Return every page of sequence ``b`` to the pool."""
        self.free.extend(reversed(self.table[b]))
        self.table[b] = []
        self.lens[b] = 0


class PagedKVCache:
    """K and V pages ``(num_pages, kv_heads, page_size, head_dim)`` on one GPU plus their page table.

    >>> cache = PagedKVCache(batch, kv_heads, head_dim, num_pages=..., page_size=256, max_seq_len=32768)
    >>> cache.append(k_prompt, v_prompt)            # (b, hk, n, d)
    >>> out = cache.decode(q, pope(cache.max_len))  # q (b, h, 1, d) at the last cached position
    """

    def __init__(self, batch: int, kv_heads: int, head_dim: int, *, num_pages: int, page_size: int = 256,
                 max_seq_len: Optional[int] = None, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if dtype not in (torch.bfloat16, torch.float16):
            raise TypeError("the paged cache holds bf16 or fp16")
        if head_dim not in (64, 96, 128):
            raise ValueError("head_dim must be 64, 96 or 128")
        self.device = torch.device(device)
        max_pages = num_pages if max_seq_len is None else -(-max_seq_len // page_size)
        self.alloc = PageAllocator(batch, num_pages, page_size, max_pages)
        self.batch, self.kv_heads, self.head_dim, self.dtype = batch, kv_heads, head_dim, dtype
        self.k_pages = torch.zeros(num_pages, kv_heads, page_size, head_dim, dtype=dtype, device=self.device)
        self.v_pages = torch.zeros_like(self.k_pages)
        self.device = self.k_pages.device   # with its index
        self.page_table = torch.zeros(batch, max_pages, dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=self.device)

    # ---- bookkeeping -------------------------------------------------------------------------------
    @property
    def page_size(self) -> int:
        return self.alloc.page_size

    @property
    def lens(self) -> List[int]:
        return list(self.alloc.lens)

    @property
    def max_len(self) -> int:
        return max(self.alloc.lens)

    def _kv_struct(self, row: int = 0) -> N.PagedKV:
        """The cache as the C ABI sees it; ``row`` > 0 = the view that starts at sequence ``row`` (a batch of one)."""
        return N.PagedKV(self.k_pages.data_ptr(), self.v_pages.data_ptr(),
                         self.page_table.data_ptr() + 4 * row * self.alloc.max_pages_per_seq, self.seq_lens.data_ptr() + 4 * row,
                         self.alloc.num_pages, self.alloc.page_size, self.alloc.max_pages_per_seq, 0)

    def _push_table(self, new_entries) -> None:
        if not new_entries:
            return
        idx = torch.tensor([[b, lp] for b, lp, _ in new_entries], dtype=torch.long)
        val = torch.tensor([pg for _, _, pg in new_entries], dtype=torch.int32)
        self.page_table[idx[:, 0].to(self.device), idx[:, 1].to(self.device)] = val.to(self.device)

    def release(self, b: int) -> None:
        """Forget sequence ``b`` and free its pages."""
        self.alloc.release(b)
        self.seq_lens[b] = 0

    # ---- the two operators -------------------------------------------------------------------------
    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v: (batch, kv_heads, n_new, head_dim) views with contiguous features; every sequence grows by n_new."""
        lib = N.load_library()
        if k.shape != v.shape or k.ndim != 4 or k.shape[0] != self.batch or k.shape[1] != self.kv_heads or k.shape[3] != self.head_dim:
            raise ValueError("k and v must be (batch, kv_heads, n_new, head_dim)")
        if k.dtype != self.dtype or v.dtype != self.dtype or k.device != self.device or v.device != self.device:
            raise TypeError("k and v must have the cache's dtype and device")
        n_new = k.shape[2]
        if n_new == 0:
            return
        k, v = N._inner_contig(k), N._inner_contig(v)
        self._push_table(self.alloc.reserve(n_new))
        a = N.KvAppendArgs(C.sizeof(N.KvAppendArgs), N._DTYPES[self.dtype], self.batch, self.kv_heads, self.head_dim, n_new, 1, 0,
                           self._kv_struct(), k.data_ptr(), N._s3(k), v.data_ptr(), N._s3(v))
        with N._on_device(self.device):
            N._check(lib.pope_b200_kv_append(C.addressof(a), N._stream_ptr(k)), "pope_b200_kv_append")
        self.alloc.advance(n_new)

    def append_to(self, b: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v: (kv_heads, n_new, head_dim) appended to sequence ``b`` only (ragged prompts)."""
        lib = N.load_library()
        if k.shape != v.shape or k.ndim != 3 or k.shape[0] != self.kv_heads or k.shape[2] != self.head_dim:
            raise ValueError("k and v must be (kv_heads, n_new, head_dim)")
        if k.dtype != self.dtype or v.dtype != self.dtype or k.device != self.device or v.device != self.device:
            raise TypeError("k and v must have the cache's dtype and device")
        n_new = k.shape[1]
        if n_new == 0:
            return
        k, v = N._inner_contig(k).unsqueeze(0), N._inner_contig(v).unsqueeze(0)
        self._push_table(self.alloc.reserve(n_new, rows=[b]))
        a = N.KvAppendArgs(C.sizeof(N.KvAppendArgs), N._DTYPES[self.dtype], 1, self.kv_heads, self.head_dim, n_new, 1, 0,
                           self._kv_struct(b), k.data_ptr(), N._s3(k), v.data_ptr(), N._s3(v))
        with N._on_device(self.device):
            N._check(lib.pope_b200_kv_append(C.addressof(a), N._stream_ptr(k)), "pope_b200_kv_append")
        self.alloc.advance(n_new, rows=[b])

    def decode(self, q: torch.Tensor, pos_emb, softmax_scale: Optional[float] = None, return_lse: bool = False):
        """q: (batch, heads, 1, head_dim); pos_emb: (freqs, bias) with at least ``max_len`` rows of freqs.
        Returns out (batch, heads, 1, head_dim) in q's dtype (and lse (batch, heads) on request)."""
        lib = N.load_library()
        freqs, bias = pos_emb
        if q.ndim != 4 or q.shape[0] != self.batch or q.shape[2] != 1 or q.shape[3] != self.head_dim or q.shape[1] % self.kv_heads != 0:
            raise ValueError("q must be (batch, heads, 1, head_dim) with heads a multiple of kv_heads")
        if q.dtype != self.dtype or q.device != self.device:
            raise TypeError("q must have the cache's dtype and device")
        r, nk = freqs.shape[-1], max(self.max_len, 1)
        if freqs.ndim != 2:
            raise ValueError("the paged decode takes a (positions, rotate_dim) table")
        if r > 0 and freqs.shape[0] < nk:
            raise ValueError("freqs must cover every cached position")
        q = N._inner_contig(q)
        freqs, bias = N._prep_embed(freqs[:nk] if r > 0 else freqs, bias, nk, r)
        out = torch.empty_like(q)
        lse = torch.empty(q.shape[0], q.shape[1], dtype=torch.float32, device=self.device)
        scale = self.head_dim ** -0.5 if softmax_scale is None else softmax_scale
        shape = N.Shape(self.batch, q.shape[1], self.kv_heads, 1, nk, self.head_dim, r, N._DTYPES[self.dtype])
        a = N.PagedDecodeArgs(C.sizeof(N.PagedDecodeArgs), float(scale), shape, N._embed_struct(freqs, bias, r), self._kv_struct(),
                              q.data_ptr(), N._s3(q), out.data_ptr(), N._s3(out), lse.data_ptr(), None, 0)
        ws = N._workspace(N.OP_DECODE_PAGED, a, self.device)
        with N._on_device(self.device):
            N._check(lib.pope_b200_attn_decode_paged(C.addressof(a), N._stream_ptr(q)), "pope_b200_attn_decode_paged")
        del ws
        return (out, lse) if return_lse else out

    # ---- for tests and debugging -------------------------------------------------------------------
    def gather(self, b: int):
        """Contiguous (kv_heads, len, head_dim) copies of sequence ``b``'s keys and values (torch indexing)."""
        n = self.alloc.lens[b]
        pages = torch.tensor(self.alloc.table[b], dtype=torch.long, device=self.device)
        k = self.k_pages[pages].permute(1, 0, 2, 3).reshape(self.kv_heads, -1, self.head_dim)[:, :n]
        v = self.v_pages[pages].permute(1, 0, 2, 3).reshape(self.kv_heads, -1, self.head_dim)[:, :n]
        return k.contiguous(), v.contiguous()
