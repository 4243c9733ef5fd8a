"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five
benchmark configurations (TinyLlama-1.1B, Llama-3-8B prefill, decode step, Llama-3-70B
KV-head-sharded, fp8-e4m3).  Index metadata is built with numpy on the host (cheap and
reproducible); K/V payloads are drawn on the device.

Byte accounting (decimal GB, per layer and per operation):
  write  : 2 * valid_tokens * (row_in + row_cache) + tokens * sizeof(slot)
  gather : 2 * sum(len) * (row_cache + row_out) + sum(ceil(len / bs)) * sizeof(idx) + seqs * sizeof(len)
where a row is num_kv_heads * head_dim elements of one token.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

SEED0 = 0x4B5658  # "KVX"


@dataclass
class Spec:
    """Static description of one configuration (global, before KV-head sharding)."""
    name: str
    io_dtype: str              # "bf16" | "f16"
    cache_dtype: str           # same, or "f8e4m3"
    layers: int
    heads: int
    dim: int
    block_size: int
    seqs: int
    len_lo: int                # sequence lengths ~ U{len_lo..len_hi}, or log-uniform
    len_hi: int
    log_uniform: bool = False
    pad_frac: float = 0.0      # fraction of slot_mapping entries set to -1
    pool_bytes: float = 0.0    # K+V, all layers, all heads; 0 = twice the needed pages
    decode: bool = False       # write = one new token per sequence (at position len-1)
    outlier_frac: float = 0.0  # fraction of elements multiplied by 50 (fp8 config)
    fixed_blocks: int = 0      # pool size in pages when the configuration states it
    index: int = 0


SPECS = {
    "c1": Spec("c1_tinyllama_1.1b", "f16", "f16", 22, 4, 64, 16, 8, 128, 128, fixed_blocks=512, index=1),
    "c2": Spec("c2_llama3_8b_prefill", "bf16", "bf16", 32, 8, 128, 16, 64, 512, 4096, pad_frac=0.10,
               pool_bytes=150e9, index=2),
    "c3": Spec("c3_decode_step", "bf16", "bf16", 32, 8, 128, 32, 512, 1, 32768, log_uniform=True, decode=True,
               index=3),
    "c4": Spec("c4_llama3_70b_head_sharded", "f16", "f16", 80, 8, 128, 16, 32, 8192, 8192, index=4),
    "c5": Spec("c5_fp8_e4m3", "bf16", "f8e4m3", 4, 16, 256, 64, 128, 2048, 2048, outlier_frac=0.001, index=5),
}

ELEM = {"bf16": 2, "f16": 2, "f32": 4, "f8e4m3": 1}


@dataclass
class Metadata:
    """Host-side index metadata of one configuration instance."""
    spec: Spec
    lens: np.ndarray            # [S] int32, full context lengths
    num_blocks: int             # pages per K (or V) tensor per layer
    table: np.ndarray           # [S, max_blocks] int32, -1 = unused
    slots: np.ndarray           # [T] int64, -1 = padding
    max_seq_len: int
    write_tokens: int           # T
    valid_tokens: int           # tokens whose slot >= 0
    gather_tokens: int          # sum(lens)
    gather_pages: int           # sum(ceil(len / bs))

    def write_bytes(self, heads: int) -> int:
        s = self.spec
        row_in = heads * s.dim * ELEM[s.io_dtype]
        row_cache = heads * s.dim * ELEM[s.cache_dtype]
        return 2 * self.valid_tokens * (row_in + row_cache) + self.write_tokens * 8

    def gather_bytes(self, heads: int) -> int:
        s = self.spec
        row_out = heads * s.dim * ELEM[s.io_dtype]
        row_cache = heads * s.dim * ELEM[s.cache_dtype]
        return 2 * self.gather_tokens * (row_cache + row_out) + self.gather_pages * 4 + s.seqs * 4


def sequence_lengths(spec: Spec, rng: np.random.Generator) -> np.ndarray:
    if spec.log_uniform:
        x = np.exp(rng.random(spec.seqs) * np.log(float(spec.len_hi)))
        return np.clip(np.rint(x), spec.len_lo, spec.len_hi).astype(np.int32)
    return rng.integers(spec.len_lo, spec.len_hi + 1, size=spec.seqs).astype(np.int32)


def build_metadata(spec: Spec, seed: Optional[int] = None, num_blocks: Optional[int] = None,
                   pool_budget_bytes: Optional[float] = None, shards: int = 1) -> Metadata:
    """Lengths, page permutation, block table and slot mapping.

    ``num_blocks`` overrides the pool size; otherwise it is ``pool_bytes`` (capped by
    ``pool_budget_bytes``, the memory one device can give to ``1/shards`` of the pool) divided
    by the page size, and never less than the pages the sequences need.
    """
    rng = np.random.default_rng(SEED0 + spec.index if seed is None else seed)
    lens = sequence_lengths(spec, rng)
    bs = spec.block_size
    need = (lens.astype(np.int64) + bs - 1) // bs
    pages_needed = int(need.sum())
    if num_blocks is None and spec.fixed_blocks:
        num_blocks = spec.fixed_blocks
    if num_blocks is None:
        page_bytes_all_heads = bs * spec.heads * spec.dim * ELEM[spec.cache_dtype]
        pool = spec.pool_bytes if spec.pool_bytes > 0 else 2.0 * pages_needed * page_bytes_all_heads * 2 * spec.layers
        if pool_budget_bytes is not None:
            pool = min(pool, pool_budget_bytes * shards)
        num_blocks = int(pool // (2 * spec.layers * page_bytes_all_heads))
    num_blocks = max(num_blocks, pages_needed)
    perm = rng.permutation(num_blocks)[:pages_needed].astype(np.int32)
    max_blocks = int(need.max())
    table = np.full((spec.seqs, max_blocks), -1, dtype=np.int32)
    starts = np.concatenate([[0], np.cumsum(need)[:-1]])
    for s in range(spec.seqs):
        table[s, : need[s]] = perm[starts[s]: starts[s] + need[s]]
    if spec.decode:
        pos = lens.astype(np.int64) - 1
        slots = table[np.arange(spec.seqs), pos // bs].astype(np.int64) * bs + pos % bs
    else:
        seq_of = np.repeat(np.arange(spec.seqs), lens)
        pos = np.concatenate([np.arange(n, dtype=np.int64) for n in lens])
        slots = table[seq_of, pos // bs].astype(np.int64) * bs + pos % bs
    if spec.pad_frac > 0:
        slots[rng.random(slots.shape[0]) < spec.pad_frac] = -1
    return Metadata(spec=spec, lens=lens, num_blocks=num_blocks, table=table, slots=slots,
                    max_seq_len=int(lens.max()), write_tokens=int(slots.shape[0]),
                    valid_tokens=int((slots >= 0).sum()), gather_tokens=int(lens.sum()),
                    gather_pages=pages_needed)


def head_range(heads: int, rank: int, world: int) -> tuple[int, int]:
    """KV heads owned by ``rank`` when the cache is sharded by head over ``world`` devices."""
    if heads % world:
        raise ValueError(f"{world} devices do not divide {heads} KV heads")
    per = heads // world
    return rank * per, (rank + 1) * per


def torch_dtype(name: str):
    import torch
    return {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "f8e4m3": torch.uint8}[name]


def draw_kv(spec: Spec, tokens: int, heads: int, device, seed: int):
    """K and V ``[tokens, heads, dim]`` ~ N(0, 1) (with x50 outliers for the fp8 config)."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = []
    for _ in range(2):
        x = torch.randn((tokens, heads, spec.dim), generator=g, device=device, dtype=torch.float32)
        if spec.outlier_frac > 0:
            m = torch.rand(x.shape, generator=g, device=device) < spec.outlier_frac
            x = torch.where(m, x * 50.0, x)
        out.append(x.to(torch_dtype(spec.io_dtype)))
        del x
    return out[0], out[1]
