"""Seeded builders of write/gather cases for the parity tests."""
from __future__ import annotations

import numpy as np

from kvx_b200 import abi

from harness import NP_OF, Case, canonical_strides, extent, f32_to_bits, random_bits

SENTINEL = {1: 0xA5, 2: 0xA5C3, 4: 0xA5C3F00D}


def sentinel_fill(n: int, code: int) -> np.ndarray:
    dt = NP_OF[code]
    return np.full(n, SENTINEL[np.dtype(dt).itemsize], dtype=dt)


def make_case(seed: int, *, layout=abi.LAYOUT_NHD, dtype=abi.DTYPE_BF16, num_blocks=8, block_size=4,
              heads=2, dim=8, pack=1, seqs=2, lens=None, max_seq_len=None, max_blocks=None,
              slot_dtype=np.int64, index_dtype=np.int32, pad_frac=0.0, oob_slots=0, bad_blocks=0,
              stride_pad=None, real_values=False, cache_dtype=None, scale_gran=abi.SCALE_NONE,
              write_all=True, tokens=None, v_pack=0) -> Case:
    """One case.  Sequences own disjoint pages drawn from a seeded permutation; the write
    batch holds every token of every sequence (sequence-major) unless ``tokens`` caps it.

    pad_frac    fraction of slots replaced by -1 (and a few by other negatives)
    oob_slots   slots pointing past the pool (block >= num_blocks): must be skipped
    bad_blocks  block-table entries replaced by -1 / >= num_blocks inside valid ranges
    stride_pad  (blk, tok, head) extra elements added to those strides (non-canonical pool); for
                HND_PACKED pools: (blk, group row, head)
    v_pack      pack factor of the V tensor of an HND_PACKED pool when it differs from K's
    """
    rng = np.random.default_rng(seed)
    geom = abi.CacheGeometry(num_blocks, block_size, heads, dim, layout, pack)
    cache_dtype = dtype if cache_dtype is None else cache_dtype
    if lens is None:
        lens = [int(rng.integers(0, 3 * block_size + 1)) for _ in range(seqs)]
    lens = list(lens)
    seqs = len(lens)
    need = [-(-n // block_size) for n in lens]
    if max_blocks is None:
        max_blocks = max(1, max(need, default=1))
    if max_seq_len is None:
        max_seq_len = max(1, max(lens, default=1))
    assert sum(need) <= num_blocks, "pool too small"
    perm = rng.permutation(num_blocks)
    table = np.full((seqs, max_blocks), -1, dtype=index_dtype)
    slots, p = [], 0
    for s, n in enumerate(lens):
        for lb in range(need[s]):
            if lb < max_blocks:
                table[s, lb] = perm[p]
            for o in range(min(block_size, n - lb * block_size)):
                slots.append(int(perm[p]) * block_size + o)
            p += 1
    slots = np.array(slots, dtype=np.int64)
    if tokens is not None:
        slots = slots[:tokens]
    T = slots.shape[0]
    if pad_frac > 0 and T:
        mask = rng.random(T) < pad_frac
        slots[mask] = -1
        neg = np.flatnonzero(mask)[:2]
        slots[neg] = [-7, -(2 ** 40)][: len(neg)] if slot_dtype == np.int64 else [-7, -12345][: len(neg)]
    for i in range(min(oob_slots, T)):
        slots[(i * 7919) % T] = num_blocks * block_size + i * block_size + (i % block_size)
    slots = slots.astype(slot_dtype)
    for i in range(bad_blocks):
        s = i % seqs
        if need[s] > 0:
            table[s, i % min(need[s], max_blocks)] = -1 if i % 2 == 0 else num_blocks + i

    if real_values:
        key = f32_to_bits(rng.standard_normal((T, heads, dim)).astype(np.float32), dtype)
        value = f32_to_bits(rng.standard_normal((T, heads, dim)).astype(np.float32), dtype)
    else:
        key, value = random_bits(rng, (T, heads, dim), dtype), random_bits(rng, (T, heads, dim), dtype)

    k_stride = v_stride = None
    n_elems = geom.elems
    geom_v = abi.CacheGeometry(num_blocks, block_size, heads, dim, layout, v_pack) if v_pack else geom
    if stride_pad is not None:
        k_stride = _padded_strides(geom, stride_pad)
        v_stride = _padded_strides(geom_v, tuple(2 * x for x in stride_pad))
        n_k, n_v = extent(geom.shape, k_stride), extent(geom_v.shape, v_stride)
    else:
        n_k = n_v = n_elems
    case = Case(geom=geom, cache_dtype=cache_dtype, io_dtype=dtype, key=key, value=value, slots=slots,
                cache_k=sentinel_fill(n_k, cache_dtype), cache_v=sentinel_fill(n_v, cache_dtype),
                k_stride=k_stride, v_stride=v_stride, table=table,
                lens=np.array(lens, dtype=index_dtype), max_seq_len=max_seq_len,
                out_k=sentinel_fill(seqs * max_seq_len * heads * dim, dtype).reshape(seqs, max_seq_len, heads, dim),
                out_v=sentinel_fill(seqs * max_seq_len * heads * dim, dtype).reshape(seqs, max_seq_len, heads, dim),
                v_pack=v_pack)
    if cache_dtype == abi.DTYPE_F8_E4M3:
        n = heads if scale_gran == abi.SCALE_PER_HEAD else 1
        case.scale_gran = scale_gran
        case.k_scale = (0.01 + rng.random(n) * 0.05).astype(np.float32)
        case.v_scale = (0.01 + rng.random(n) * 0.05).astype(np.float32)
    return case


def _padded_strides(geom: abi.CacheGeometry, pad) -> list[int]:
    """Strides of an NHD/HND pool whose head, token and block pitches are padded (multiples
    given in elements), keeping dim contiguous."""
    blk_pad, tok_pad, head_pad = pad
    D, H, bs = geom.head_dim, geom.num_kv_heads, geom.block_size
    if geom.layout == abi.LAYOUT_NHD:
        s_head = D + head_pad
        s_tok = H * s_head + tok_pad
        s_blk = bs * s_tok + blk_pad
        return [s_blk, s_tok, s_head, 1]
    if geom.layout == abi.LAYOUT_HND:
        s_tok = D + tok_pad
        s_head = bs * s_tok + head_pad
        s_blk = H * s_head + blk_pad
        return [s_blk, s_head, s_tok, 1]
    if geom.layout == abi.LAYOUT_HND_PACKED:
        s_row = bs * geom.pack + tok_pad          # one pack group of every token of the page
        s_head = (D // geom.pack) * s_row + head_pad
        s_blk = H * s_head + blk_pad
        return [s_blk, s_head, s_row, geom.pack, 1]
    raise ValueError("padded strides: unknown layout")


def expected_write_numpy(case: Case):
    """Independent numpy statement of the canonical-stride write, used to cross-check the C
    checker itself (follows the expected-value loops of the reference's kernel test,
    tests/kvx_kernel_test.cu:264-301 for NHD and :415-446 for HND)."""
    g = case.geom
    assert case.k_stride is None and case.cache_dtype == case.io_dtype
    k = case.cache_k.copy().reshape(g.shape)
    v = case.cache_v.copy().reshape(g.shape)
    for t, slot in enumerate(case.slots.tolist()):
        if slot < 0:
            continue
        b, o = divmod(slot, g.block_size)
        if b >= g.num_blocks:
            continue
        for dst, src in ((k, case.key), (v, case.value)):
            if g.layout == abi.LAYOUT_NHD:
                dst[b, o] = src[t]
            elif g.layout == abi.LAYOUT_HND:
                dst[b, :, o, :] = src[t]
            else:
                dst[b, :, :, o, :] = src[t].reshape(g.num_kv_heads, g.head_dim // g.pack, g.pack)
    return k.reshape(-1), v.reshape(-1)


def expected_gather_numpy(case: Case, cache_k: np.ndarray, cache_v: np.ndarray):
    """Independent numpy statement of the gather (tests/kvx_kernel_test.cu:749-777)."""
    g = case.geom
    assert case.k_stride is None and case.cache_dtype == case.io_dtype
    outs = []
    for pool, out0 in ((cache_k, case.out_k), (cache_v, case.out_v)):
        pool = pool.reshape(g.shape)
        out = out0.copy()
        for s in range(case.table.shape[0]):
            for tok in range(min(int(case.lens[s]), case.max_seq_len)):
                lb, o = divmod(tok, g.block_size)
                if lb >= case.table.shape[1]:
                    continue
                b = int(case.table[s, lb])
                if b < 0 or b >= g.num_blocks:
                    continue
                if g.layout == abi.LAYOUT_NHD:
                    out[s, tok] = pool[b, o]
                elif g.layout == abi.LAYOUT_HND:
                    out[s, tok] = pool[b, :, o, :]
                else:
                    out[s, tok] = pool[b, :, :, o, :].reshape(g.num_kv_heads, g.head_dim)
        outs.append(out)
    return outs[0], outs[1]


def to_ragged(case: Case, indptr_dtype=np.int32, truncate=()) -> Case:
    """The same gather expressed with a RAGGED table: one page id per cached token, taken from
    the PACKED table (KVX_SPEC.md:108-114).  ``truncate`` lists sequences whose token list is
    cut to half their length (the gather must then stop there)."""
    import dataclasses
    bs = case.geom.block_size
    ids, counts = [], []
    for s in range(case.table.shape[0]):
        n = int(min(max(int(case.lens[s]), 0), case.table.shape[1] * bs))
        if s in truncate:
            n //= 2
        ids.extend(int(case.table[s, t // bs]) for t in range(n))
        counts.append(n)
    indptr = np.concatenate([[0], np.cumsum(counts)]).astype(indptr_dtype)
    return dataclasses.replace(case, ragged=np.array(ids, dtype=case.table.dtype), indptr=indptr)


def damage_indptr(case: Case, seed: int) -> Case:
    """A RAGGED case whose indptr no longer fits its index array: one entry negative, one beyond
    the end of the array.  Tokens whose entry would lie outside the array must be skipped."""
    import dataclasses
    rng = np.random.default_rng(seed)
    indptr = case.indptr.copy()
    n = indptr.shape[0]
    total = int(case.ragged.shape[0])
    if n > 2:
        indptr[int(rng.integers(1, n - 1))] = -3
    indptr[n - 1] = total + 1000        # the last sequence claims more entries than exist
    if n > 3:
        indptr[int(rng.integers(1, n - 1))] = total + 7
    return dataclasses.replace(case, indptr=indptr)


def expected_gather_ragged_numpy(case: Case, cache_k: np.ndarray, cache_v: np.ndarray):
    """Independent numpy statement of the RAGGED gather (NHD / HND canonical pools)."""
    g = case.geom
    outs = []
    for pool, out0 in ((cache_k, case.out_k), (cache_v, case.out_v)):
        pool = pool.reshape(g.shape)
        out = out0.copy()
        for s in range(case.indptr.shape[0] - 1):
            first, count = int(case.indptr[s]), int(case.indptr[s + 1] - case.indptr[s])
            for tok in range(min(int(case.lens[s]), case.max_seq_len, count)):
                if first < 0 or first + tok >= case.ragged.shape[0]:
                    continue  # damaged indptr: the entry would lie outside the index array
                b = int(case.ragged[first + tok])
                if b < 0 or b >= g.num_blocks:
                    continue
                o = tok % g.block_size
                out[s, tok] = pool[b, o] if g.layout == abi.LAYOUT_NHD else pool[b, :, o, :]
        outs.append(out)
    return outs[0], outs[1]


def to_kv_offsets(case: Case, cache_k: np.ndarray, cache_v: np.ndarray, seed: int = 0, secondary_frac: float = 0.3,
                  with_secondary: bool = True, unused: int = 0x7FFFFFFF) -> Case:
    """The same gather expressed the TensorRT-LLM way (KVX_SPEC.md:116-122): every K page and
    every V page of the canonical pools ``cache_k`` / ``cache_v`` becomes one block of a
    primary or (for a seeded fraction of the blocks) a secondary pool, at a seeded position;
    the int32 table ``[S, 1, 2, max_blocks]`` holds the pool offsets, bit 31 set for the
    secondary pool.  Table entries that PACKED marks invalid get ``unused`` (an offset beyond
    the pool).  With ``with_secondary=False`` the secondary pool is withheld, so its entries
    must be skipped.  The gather result must equal the PACKED one (where pages are present)."""
    import dataclasses
    g = case.geom
    assert case.k_stride is None and g.layout in (abi.LAYOUT_NHD, abi.LAYOUT_HND)
    rng = np.random.default_rng(seed)
    NB = g.num_blocks
    page = g.elems // NB                      # elements per page
    pages = np.concatenate([cache_k.reshape(NB, page), cache_v.reshape(NB, page)])  # K pages then V pages
    in_secondary = rng.random(2 * NB) < secondary_frac
    pools, where = [], np.zeros(2 * NB, dtype=np.uint32)
    for flag in (False, True):
        ids = np.flatnonzero(in_secondary == flag)
        spots = rng.permutation(2 * NB)[: len(ids)]     # scattered over a pool of 2 NB blocks
        pool = sentinel_fill(2 * NB * page, case.cache_dtype).reshape(2 * NB, page)
        pool[spots] = pages[ids]
        where[ids] = spots.astype(np.uint32) | (np.uint32(0x80000000) if flag else np.uint32(0))
        pools.append(pool.reshape(-1))
    S, M = case.table.shape
    table = np.full((S, 1, 2, M), unused, dtype=np.uint32)
    for s in range(S):
        for lb in range(M):
            b = int(case.table[s, lb])
            if 0 <= b < NB:
                table[s, 0, 0, lb] = where[b]
                table[s, 0, 1, lb] = where[NB + b]
    geom = abi.CacheGeometry(2 * NB, g.block_size, g.num_kv_heads, g.head_dim, g.layout, g.pack)
    return dataclasses.replace(case, geom=geom, kv_offsets=table.view(np.int32), pool_primary=pools[0],
                               pool_secondary=pools[1] if with_secondary else None,
                               pool_block_bytes=page * pools[0].dtype.itemsize,
                               lens=case.lens.astype(np.int32), table=case.table.astype(np.int32),
                               keep=[in_secondary])


def expected_without_secondary(packed: Case, off: Case, packed_k: np.ndarray, packed_v: np.ndarray):
    """Expected KV_OFFSETS gather when the secondary pool is withheld: the PACKED result, with
    the rows whose K (resp. V) page went to the secondary pool left as they were."""
    in_secondary = off.keep[0]
    NB, bs = packed.geom.num_blocks, packed.geom.block_size
    ek, ev = packed_k.copy(), packed_v.copy()
    for s in range(packed.table.shape[0]):
        for tok in range(min(int(packed.lens[s]), packed.max_seq_len)):
            lb = tok // bs
            if lb >= packed.table.shape[1]:
                continue
            b = int(packed.table[s, lb])
            if not 0 <= b < NB:
                continue
            if in_secondary[b]:
                ek[s, tok] = packed.out_k[s, tok]
            if in_secondary[NB + b]:
                ev[s, tok] = packed.out_v[s, tok]
    return ek, ev


def to_varlen(case: Case, indptr_dtype=np.int32, gap: int = 0, short=(), rows_cut: int = 0) -> Case:
    """The same gather into un-padded ``[rows, H, D]`` outputs: sequence s starts at row
    ``out_indptr[s]``.  ``gap`` leaves unused rows between sequences, ``short`` lists sequences
    given half the rows they need (the gather must stop there), ``rows_cut`` removes rows from
    the end of the tensors (the gather must not write past them)."""
    import dataclasses
    H, D = case.geom.num_kv_heads, case.geom.head_dim
    counts = []
    for s in range(case.table.shape[0]):
        n = int(min(max(int(case.lens[s]), 0), case.max_seq_len))
        counts.append((n // 2 if s in short else n) + gap)
    indptr = np.concatenate([[0], np.cumsum(counts)]).astype(indptr_dtype)
    rows = max(0, int(indptr[-1]) - rows_cut)
    return dataclasses.replace(case, out_indptr=indptr,
                               out_k=sentinel_fill(rows * H * D, case.io_dtype).reshape(rows, H, D),
                               out_v=sentinel_fill(rows * H * D, case.io_dtype).reshape(rows, H, D))


def expected_varlen_from_padded(case: Case, padded_k: np.ndarray, padded_v: np.ndarray, gap: int = 0):
    """Expected un-padded outputs derived from the PADDED gather result of the same case: row
    out_indptr[s] + tok takes padded[s, tok] where the padded gather wrote it (tok below the
    sequence length), limited to the rows of the sequence and of the tensor."""
    ek, ev = case.out_k.copy(), case.out_v.copy()
    rows = ek.shape[0]
    for s in range(case.table.shape[0]):
        first, room = int(case.out_indptr[s]), int(case.out_indptr[s + 1] - case.out_indptr[s])
        n = min(max(int(case.lens[s]), 0), case.max_seq_len, room, max(0, rows - first))
        ek[first:first + n] = padded_k[s, :n]
        ev[first:first + n] = padded_v[s, :n]
    return ek, ev


def to_pitched(case: Case, key_extra: int, value_extra: int, seed: int = 0) -> Case:
    """The same write with key / value token rows ``heads * dim + extra`` elements apart, as
    slices of a fused projection output are; the gaps hold random bits that must not be read
    into the cache."""
    import dataclasses
    rng = np.random.default_rng(seed)
    hd = case.geom.num_kv_heads * case.geom.head_dim
    out = {}
    for name, extra in (("key", key_extra), ("value", value_extra)):
        src = getattr(case, name).reshape(case.T, hd)
        wide = random_bits(rng, (case.T, hd + extra), case.io_dtype)
        wide[:, :hd] = src
        out[name] = wide
        out[name + "_pitch"] = hd + extra
    return dataclasses.replace(case, **out)


def reorder_tokens(case: Case, order: np.ndarray) -> Case:
    """The same case with the write batch's tokens taken in ``order`` (a permutation or a
    selection): rows and slots move together, so the pages end up the same for a permutation."""
    import dataclasses
    order = np.asarray(order, dtype=np.int64)
    return dataclasses.replace(case, key=case.key[order].copy(), value=case.value[order].copy(),
                               slots=case.slots[order].copy())
