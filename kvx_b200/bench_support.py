"""Device-side set-up shared by ``bench.py`` and the full-size tests: allocate the page pool of
a configuration, place its inputs in HBM, and build the per-layer ABI descriptors once."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import tempfile
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from . import abi, workloads
from ._lib import lib

DTYPE_CODE = {"bf16": abi.DTYPE_BF16, "f16": abi.DTYPE_F16, "f32": abi.DTYPE_F32, "f8e4m3": abi.DTYPE_F8_E4M3}


@dataclass
class DeviceWorkload:
    """One rank's share (its KV heads) of a configuration, resident on its device."""
    meta: workloads.Metadata
    heads: int                      # local KV heads
    layers: int
    pool: "torch.Tensor"            # uint8, all layers, K and V
    key: "torch.Tensor"             # [T, heads, dim]
    value: "torch.Tensor"
    slots: "torch.Tensor"           # [T] int64
    table: "torch.Tensor"           # [S, max_blocks] int32
    lens: "torch.Tensor"            # [S] int32
    out_k: "torch.Tensor"           # [S, Lmax, heads, dim]
    out_v: "torch.Tensor"
    k_scale: Optional["torch.Tensor"] = None
    v_scale: Optional["torch.Tensor"] = None
    caches: list = field(default_factory=list)   # per layer abi.CacheDesc
    write: Optional[abi.WriteDesc] = None
    gather: Optional[abi.GatherDesc] = None
    ks_desc: Optional[abi.ScaleDesc] = None
    vs_desc: Optional[abi.ScaleDesc] = None
    layout: str = "nhd"             # "nhd" | "hnd" | "packed" (K and V in 16-byte pack groups) | "paged"
                                    # (K in 16-byte pack groups, V [blocks, heads, dim, block_size])

    @property
    def write_bytes(self) -> int:
        return self.meta.write_bytes(self.heads)

    @property
    def gather_bytes(self) -> int:
        return self.meta.gather_bytes(self.heads)

    def tensor_bytes(self) -> int:
        s = self.meta.spec
        return self.meta.num_blocks * s.block_size * self.heads * s.dim * workloads.ELEM[s.cache_dtype]

    def packs(self) -> tuple[int, int]:
        """Pack factor (elements per pack group) of the K and of the V tensor; 0 = not packed."""
        x = 16 // workloads.ELEM[self.meta.spec.cache_dtype]
        return {"nhd": (0, 0), "hnd": (0, 0), "packed": (x, x), "paged": (x, 1)}[self.layout]

    def layer_pages(self, layer: int):
        """(K pages, V pages) of one layer, each a view of the pool with the axes in the order
        (block, token in block, head, ...dim): [num_blocks, block_size, heads, dim] for NHD (as it
        lies in memory) and HND (permuted), [num_blocks, block_size, heads, dim / pack, pack] for the
        packed layouts.  Indexing the first two axes gives one token's row whatever the layout."""
        import torch
        s = self.meta.spec
        n = self.tensor_bytes()
        nb, bs, H, D = self.meta.num_blocks, s.block_size, self.heads, s.dim
        dt = workloads.torch_dtype(s.cache_dtype)
        out = []
        for which, pack in zip((0, 1), self.packs()):
            flat = self.pool[(2 * layer + which) * n:(2 * layer + which + 1) * n].view(dt)
            if self.layout == "nhd":
                out.append(flat.view(nb, bs, H, D))
            elif self.layout == "hnd":
                out.append(flat.view(nb, H, bs, D).permute(0, 2, 1, 3))
            else:
                out.append(flat.view(nb, H, D // pack, bs, pack).permute(0, 3, 1, 2, 4))
        return out[0], out[1]


def setup_device_workload(spec: workloads.Spec, rank: int = 0, world: int = 1, layers: Optional[int] = None,
                          pool_gb: Optional[float] = None, num_blocks: Optional[int] = None,
                          reserve_bytes: float = 6e9, seed: Optional[int] = None,
                          layout: str = "nhd") -> DeviceWorkload:
    """Allocate and fill one rank's share.  The pool takes ``spec.pool_bytes / world`` or what
    the device can spare (free memory minus inputs, outputs and ``reserve_bytes``).  ``layout``
    is the page layout the descriptors announce (see :class:`DeviceWorkload`)."""
    import torch
    dev = torch.device("cuda", torch.cuda.current_device())
    layers = spec.layers if layers is None else layers
    h0, h1 = workloads.head_range(spec.heads, rank, world)
    heads = h1 - h0
    e_io, e_c = workloads.ELEM[spec.io_dtype], workloads.ELEM[spec.cache_dtype]

    # Size everything else first, then give the pool what is left.
    probe = workloads.build_metadata(spec, seed=seed, num_blocks=1)
    T, S, Lmax = probe.write_tokens, spec.seqs, probe.max_seq_len
    io_bytes = 2 * T * heads * spec.dim * e_io + 2 * S * Lmax * heads * spec.dim * e_io
    free, _total = torch.cuda.mem_get_info()
    budget = free - io_bytes - reserve_bytes - 2 * T * spec.heads * spec.dim * 4  # f32 scratch while drawing K/V
    if pool_gb is not None:
        budget = min(budget, pool_gb * 1e9)
    scale_layers = layers / spec.layers
    meta = workloads.build_metadata(spec, seed=seed, num_blocks=num_blocks,
                                    pool_budget_bytes=max(budget, 0) / scale_layers, shards=world)
    page_local = spec.block_size * heads * spec.dim * e_c
    # A configuration whose pages for all layers cannot fit (the decode step's full contexts)
    # runs on as many layers as do fit; the count is reported with the result.
    while layers > 1 and 2 * layers * meta.num_blocks * page_local > budget:
        layers -= 1
    pool_bytes = 2 * layers * meta.num_blocks * page_local
    if pool_bytes > budget + 1:
        raise RuntimeError(f"page pool of {pool_bytes / 1e9:.1f} GB does not fit ({budget / 1e9:.1f} GB available)")
    pool = torch.empty(pool_bytes, dtype=torch.uint8, device=dev)

    key_all, value_all = workloads.draw_kv(spec, T, spec.heads, dev, workloads.SEED0 + 100 + spec.index)
    key = key_all[:, h0:h1].contiguous()
    value = value_all[:, h0:h1].contiguous()
    del key_all, value_all
    torch.cuda.empty_cache()

    dw = DeviceWorkload(meta=meta, heads=heads, layers=layers, pool=pool, key=key, value=value,
                        slots=torch.from_numpy(meta.slots).to(dev), table=torch.from_numpy(meta.table).to(dev),
                        lens=torch.from_numpy(meta.lens).to(dev),
                        out_k=torch.empty((S, Lmax, heads, spec.dim), dtype=key.dtype, device=dev),
                        out_v=torch.empty((S, Lmax, heads, spec.dim), dtype=key.dtype, device=dev), layout=layout)
    build_descriptors(dw)
    return dw


def build_descriptors(dw: DeviceWorkload) -> None:
    """Per-layer cache descriptors plus one write and one gather descriptor."""
    s, m = dw.meta.spec, dw.meta
    code = {"nhd": abi.LAYOUT_NHD, "hnd": abi.LAYOUT_HND, "packed": abi.LAYOUT_HND_PACKED,
            "paged": abi.LAYOUT_HND_PACKED}[dw.layout]
    pack_k, pack_v = dw.packs()
    geom = abi.CacheGeometry(m.num_blocks, s.block_size, dw.heads, s.dim, code, max(pack_k, 1))
    geom_v = abi.CacheGeometry(m.num_blocks, s.block_size, dw.heads, s.dim, code, max(pack_v, 1))
    tensor_bytes = geom.elems * workloads.ELEM[s.cache_dtype]
    base = dw.pool.data_ptr()
    code_c, code_io = DTYPE_CODE[s.cache_dtype], DTYPE_CODE[s.io_dtype]
    dw.caches = []
    for l in range(dw.layers):
        c = abi.cache_desc(geom, code_c, base + (2 * l) * tensor_bytes, base + (2 * l + 1) * tensor_bytes)
        if pack_v != pack_k:
            c.v = abi.tensor_desc(base + (2 * l + 1) * tensor_bytes, code_c, geom_v.shape, None, code)
        dw.caches.append(c)
    if s.cache_dtype == "f8e4m3":
        from . import ops
        dw.k_scale, dw.v_scale = ops.compute_kv_scales(dw.key, dw.value, per_head=True)
        dw.ks_desc = abi.scale_desc(dw.k_scale.data_ptr(), abi.SCALE_PER_HEAD, dw.heads)
        dw.vs_desc = abi.scale_desc(dw.v_scale.data_ptr(), abi.SCALE_PER_HEAD, dw.heads)
    dw.write = abi.write_desc(m.write_tokens, dw.heads, s.dim, code_io, dw.key.data_ptr(), dw.value.data_ptr(),
                              abi.DTYPE_S64, dw.slots.data_ptr(), k_scale=dw.ks_desc, v_scale=dw.vs_desc)
    dw.gather = abi.gather_desc(s.seqs, m.max_seq_len, dw.heads, s.dim, code_io, dw.out_k.data_ptr(),
                                dw.out_v.data_ptr(), abi.DTYPE_S32, dw.table.data_ptr(), m.table.shape[1],
                                dw.lens.data_ptr())


def launch_write(dw: DeviceWorkload, layer: int, stream: int) -> None:
    st = lib().kvx_launch_write_kv(C.byref(dw.caches[layer]), C.byref(dw.write), stream)
    if st != abi.STATUS_OK:
        raise RuntimeError(f"kvx_launch_write_kv status {st}")


def launch_gather(dw: DeviceWorkload, layer: int, stream: int) -> None:
    if dw.ks_desc is not None:
        st = lib().kvx_launch_gather_kv_f8e4m3(C.byref(dw.caches[layer]), C.byref(dw.gather), C.byref(dw.ks_desc),
                                               C.byref(dw.vs_desc), stream)
    else:
        st = lib().kvx_launch_gather_kv(C.byref(dw.caches[layer]), C.byref(dw.gather), stream)
    if st != abi.STATUS_OK:
        raise RuntimeError(f"kvx_launch_gather_kv status {st}")


SENTINEL = 0x5A  # byte pattern the gather outputs are filled with before a verified run


def fill_sentinel(dw: DeviceWorkload) -> None:
    """Prepares a workload for :func:`verify_layer`: the page pool becomes a position-dependent
    pattern (64-bit word i holds i, so no two rows of the pool look alike and a page taken from
    the wrong place shows) and every byte of the gather outputs becomes ``SENTINEL``."""
    import torch
    words = dw.pool.view(torch.int64)
    step = 1 << 28
    for w0 in range(0, words.shape[0], step):
        w1 = min(w0 + step, words.shape[0])
        torch.arange(w0, w1, dtype=torch.int64, device=words.device, out=words[w0:w1])
    dw.out_k.view(torch.uint8).fill_(SENTINEL)
    dw.out_v.view(torch.uint8).fill_(SENTINEL)


def _all_sentinel(rows) -> bool:
    return bool((rows == SENTINEL).all())


def _bits(t):
    """The tensor's elements as integers of the same width: comparisons must see bit patterns
    (the fill pattern and the sentinel contain NaN encodings, which never compare equal as floats)."""
    import torch
    return t.contiguous().view({1: torch.uint8, 2: torch.int16, 4: torch.int32}[t.element_size()])


def verify_layer(dw: DeviceWorkload, layer: int) -> dict:
    """Byte check of one layer of a workload that was prepared with :func:`fill_sentinel`,
    then written, then gathered into ``dw.out_k`` / ``dw.out_v``.  Torch index operations on the
    device only: an independent statement of the write and of the gather, for every page layout
    :func:`build_descriptors` knows, that needs no CPU copy of the data.

    * write_rows: rows of the pool addressed by valid slots hold the input rows (an fp8 cache:
      within half an e4m3 step of ``input / scale``),
    * untouched_pages: every other row of the layer's K and V tensors still holds the fill pattern,
    * gather_live: output rows below a sequence's length hold what the pages hold at
      ``table[s, p // block_size] * block_size + p % block_size`` (an fp8 cache: those bytes
      dequantised with the head's scale and rounded to the output type),
    * gather_dead: output rows at or past the length still hold the sentinel.
    """
    import torch
    s, m = dw.meta.spec, dw.meta
    dev = dw.pool.device
    fp8 = s.cache_dtype == "f8e4m3"
    bs_, nb = s.block_size, m.num_blocks
    row_io = dw.heads * s.dim * workloads.ELEM[s.io_dtype]
    kp, vp = dw.layer_pages(layer)
    slots = dw.slots
    valid = slots >= 0
    idx = slots[valid]
    inside = idx < nb * bs_                       # a slot beyond the pool is skipped by the write
    blk, off = (idx // bs_)[inside], (idx % bs_)[inside]
    vi = valid.nonzero().flatten()[inside]         # token numbers of the rows that must have landed

    def rows_of(pages, b, o):                      # [n, heads * dim] elements of the given (block, offset) rows
        return pages[b, o].reshape(b.shape[0], -1)

    res = {}
    ok = True
    for pages, src, scale in ((kp, dw.key, dw.k_scale), (vp, dw.value, dw.v_scale)):
        if fp8:
            n = min(int(vi.shape[0]), 1 << 15)
            got = rows_of(pages, blk[:n], off[:n]).view(torch.float8_e4m3fn).float().view(n, dw.heads, s.dim)
            want = (src[vi[:n]].float() / scale[None, :, None]).clamp(-448.0, 448.0)
            ulp = torch.clamp(want.abs(), min=2.0 ** -6) * 2.0 ** -3   # at least the e4m3 step at |want|
            ok = ok and bool(((got - want).abs() <= 0.5 * ulp * 1.0001 + 2.0 ** -10).all())
        else:
            for t0 in range(0, vi.shape[0], 1 << 17):
                sl = slice(t0, t0 + (1 << 17))
                ok = ok and bool(torch.equal(_bits(rows_of(pages, blk[sl], off[sl])),
                                             _bits(src[vi[sl]].reshape(-1, dw.heads * s.dim))))
    res["write_rows"] = ok

    # untouched rows, a slab of blocks at a time: the fill pattern is rebuilt for the slab and seen
    # through the same permutation of axes as the pages
    touched = torch.zeros(nb * bs_, dtype=torch.bool, device=dev)
    touched[idx[inside]] = True
    touched = touched.view(nb, bs_)
    page_words = kp[0].numel() * kp.element_size() // 8
    slab = max(1, int(2.5e8 // (page_words * 8)))
    ok = True
    for which, pages in ((0, kp), (1, vp)):
        first_word = ((2 * layer + which) * dw.tensor_bytes()) // 8
        for b0 in range(0, nb, slab):
            b1 = min(nb, b0 + slab)
            free = ~touched[b0:b1]
            if not bool(free.any()):
                continue
            want = torch.arange(first_word + b0 * page_words, first_word + b1 * page_words, dtype=torch.int64,
                                device=dev)
            # same shape games as layer_pages, on 8-byte words viewed as cache elements
            want_pages = _like_pages(dw, want.view(kp.dtype), b1 - b0, which)
            ok = ok and bool(torch.equal(_bits(pages[b0:b1][free]), _bits(want_pages[free])))
            del want, want_pages
    res["untouched_pages"] = ok
    del touched

    S, Lmax = s.seqs, m.max_seq_len
    lens = dw.lens.to(torch.int64)
    ok_b = dw.out_k.view(torch.uint8).view(S, Lmax, row_io)
    ov_b = dw.out_v.view(torch.uint8).view(S, Lmax, row_io)
    step = max(1, int(2.5e8 // (Lmax * row_io)))
    pos = torch.arange(Lmax, device=dev)
    dead_ok, live_ok = True, True
    block = dw.table.to(torch.int64)
    for s0 in range(0, S, step):
        live = pos[None, :] < lens[s0:s0 + step, None]
        dead_ok = dead_ok and _all_sentinel(ok_b[s0:s0 + step][~live]) and _all_sentinel(ov_b[s0:s0 + step][~live])
        sq, pp = live.nonzero(as_tuple=True)
        b_of = block[s0 + sq, pp // bs_]
        for out_b, pages, scale in ((ok_b, kp, dw.k_scale), (ov_b, vp, dw.v_scale)):
            got = out_b[s0:s0 + step][live]
            held = rows_of(pages, b_of, pp % bs_)
            if fp8:
                want = held.view(torch.float8_e4m3fn).float().view(-1, dw.heads, s.dim) * scale[None, :, None]
                want = want.to(workloads.torch_dtype(s.io_dtype))
            else:
                want = held
            live_ok = live_ok and bool(torch.equal(got, want.reshape(got.shape[0], -1).contiguous().view(torch.uint8)))
            del got, want, held
    res["gather_live"] = live_ok
    res["gather_dead"] = dead_ok
    res["ok"] = all(res.values())
    return res


def _like_pages(dw: DeviceWorkload, flat, blocks: int, which: int):
    """``flat`` (the elements of ``blocks`` whole pages of the K (which = 0) or V (1) tensor, as
    they lie in memory) with the axes in the order :meth:`DeviceWorkload.layer_pages` uses."""
    s = dw.meta.spec
    bs_, H, D = s.block_size, dw.heads, s.dim
    pack = dw.packs()[which]
    if dw.layout == "nhd":
        return flat.view(blocks, bs_, H, D)
    if dw.layout == "hnd":
        return flat.view(blocks, H, bs_, D).permute(0, 2, 1, 3)
    return flat.view(blocks, H, D // pack, bs_, pack).permute(0, 3, 1, 2, 4)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a timed region
    runs (read-only queries; nothing is set)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 100):
        self.gpu, self.period, self.proc, self.path = gpu_index, period_ms, None, None

    def start(self) -> None:
        fd, self.path = tempfile.mkstemp(prefix="kvx_clocks_", suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
            return
        # nvidia-smi needs a moment to start; wait for its first line so that short runs are sampled too
        import time
        deadline = time.time() + 3.0
        while time.time() < deadline and os.path.getsize(self.path) == 0 and self.proc.poll() is None:
            time.sleep(0.02)

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, mx, power = [], set(), None, []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    clocks.append(float(f[1])); mx = float(f[2]); power.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        if clocks:
            # "under load" = samples in the upper half of the power range seen
            out.update(sm_mhz=float(np.median(clocks)), sm_max_mhz=mx, reasons=sorted(reasons),
                       samples=len(clocks), power_w_max=max(power))
        return out
