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

    @property
    def write_bytes(self) -> int:
        return self.meta.write_bytes(self.heads)

    @property
    def gather_bytes(self) -> int:
        return self.meta.gather_bytes(self.heads)

    def layer_pages(self, layer: int):
        """(K pages, V pages) of one layer as [num_blocks, block_size, heads, dim] views."""
        import torch
        s = self.meta.spec
        n = self.meta.num_blocks * s.block_size * self.heads * s.dim * workloads.ELEM[s.cache_dtype]
        shape = (self.meta.num_blocks, s.block_size, self.heads, s.dim)
        dt = workloads.torch_dtype(s.cache_dtype)
        k = self.pool[(2 * layer) * n:(2 * layer + 1) * n].view(dt).view(shape)
        v = self.pool[(2 * layer + 1) * n:(2 * layer + 2) * n].view(dt).view(shape)
        return k, v


def setup_device_workload(spec: workloads.Spec, rank: int = 0, world: int = 1, layers: Optional[int] = None,
                          pool_gb: Optional[float] = None, num_blocks: Optional[int] = None,
                          reserve_bytes: float = 6e9, seed: Optional[int] = None) -> DeviceWorkload:
    """Allocate and fill one rank's share.  The pool takes ``spec.pool_bytes / world`` or what
    the device can spare (free memory minus inputs, outputs and ``reserve_bytes``)."""
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
                        out_v=torch.empty((S, Lmax, heads, spec.dim), dtype=key.dtype, device=dev))
    build_descriptors(dw)
    return dw


def build_descriptors(dw: DeviceWorkload) -> None:
    """Per-layer cache descriptors plus one write and one gather descriptor."""
    s, m = dw.meta.spec, dw.meta
    geom = abi.CacheGeometry(m.num_blocks, s.block_size, dw.heads, s.dim)
    tensor_bytes = geom.elems * workloads.ELEM[s.cache_dtype]
    base = dw.pool.data_ptr()
    code_c, code_io = DTYPE_CODE[s.cache_dtype], DTYPE_CODE[s.io_dtype]
    dw.caches = [abi.cache_desc(geom, code_c, base + (2 * l) * tensor_bytes, base + (2 * l + 1) * tensor_bytes)
                 for l in range(dw.layers)]
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
