/*
 * Paged KV-cache write / gather for NVIDIA B200 (sm_100a): launch layer + kernels, one
 * self-contained translation unit with C linkage (needs only kvx_abi.h, kvx_paged_kv.h
 * and the CUDA runtime, so it can be added to another project's source list as is).
 *
 * The work is pure data movement bounded by HBM bandwidth, so the kernels are organised
 * around three things only: 16-byte coalesced accesses, many independent loads in flight
 * per thread before the first store, and no wasted threads on padding.
 *
 *   write, vector tier   kvx_write_rows_kernel     one CTA = a tile of consecutive tokens;
 *                        slot -> destination byte offsets are resolved once per token into
 *                        shared memory, then all threads stream the tile's 16-byte vectors
 *                        (4 K + 4 V loads in flight per thread, streaming cache hints).
 *   gather, vector tier  kvx_gather_pages_kernel   persistent CTAs; every CTA compacts the
 *                        ragged (sequence, page) rectangle with a shared-memory prefix sum
 *                        over ceil(len / block_size), then each warp copies whole page
 *                        chunks (contiguous on both sides for NHD) 8 vectors deep.
 *   gather, bulk tier    kvx_gather_bulk_kernel    same decomposition, but a page chunk is
 *                        staged global -> shared -> global with cp.async.bulk (the TMA
 *                        engine), one elected thread per ring of stages.
 *   packed pages         kvx_write_packed_kernel / kvx_gather_packed_kernel: HND_PACKED pages whose
 *                        pack group is 2 .. 16 bytes (K and V each with its own pack factor)
 *                        are a transposition, in units of the group, of the dense token rows;
 *                        it is done in registers with warp shuffles between full 16- and
 *                        32-byte accesses on both sides, the write after cutting its tokens
 *                        into runs of consecutive slots -- or, with K and V in 16-byte groups
 *                        (kvx_write_packed_lines_kernel), after sorting them into the 8-slot
 *                        windows of the pages' 128-byte lines.
 *   fp8-e4m3             quantise-on-write / dequantise-on-gather variants of the vector tiers
 *                        plus the absmax -> scale reduction.
 *   generic tier         one element per thread for layouts, head sizes or alignments the
 *                        other tiers cannot take (odd head_dim, misaligned tensors, ...).
 *
 * Semantics (which element goes where, what is skipped) follow the reference kernels:
 * kernels/kvx_paged_kv.cu:54-75 (offsets), :98-123 (write), :232-266 (gather).
 */
#include "kvx_paged_kv.h"

#include "kvx_pages.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <numeric>

namespace {

// ------------------------------------------------------------------ tunables ----------

// Written by kvx_b200_set_option, read by the launchers, possibly from different host threads:
// every field is an atomic, read and written with relaxed ordering (a launch sees the old or the
// new value of a knob, never a torn one).
struct Options {
  std::atomic<int64_t> write_vecs_per_cta{1024};  // 16-byte vectors of K (and of V) one write CTA moves
  std::atomic<int64_t> write_unroll{4};           // vectors of K and of V in flight per thread (1,2,4)
  std::atomic<int64_t> gather_path{2};            // 0 = CTA-granular register copy, 1 = cp.async.bulk staging, 2 = warp-granular
  std::atomic<int64_t> gather_tile_bytes{16384};  // bytes of K (and of V) one CTA moves per work item (path 0)
  std::atomic<int64_t> gather_ctas_per_sm{256};   // most CTAs launched per SM (register paths; 4 are resident at a time)
  std::atomic<int64_t> gather_part_bytes{4096};   // span one warp copies per work item (one unrolled iteration)
  std::atomic<int64_t> bulk_stage_bytes{16384};   // bytes per shared-memory stage (bulk path)
  std::atomic<int64_t> bulk_stages{4};            // stages per pipe (bulk path)
  std::atomic<int64_t> bulk_pipes{3};             // pipes (elected threads) per CTA (bulk path)
  std::atomic<int64_t> bulk_lag{2};               // loads a pipe keeps in flight ahead of its stores
  std::atomic<int64_t> bulk_ctas_per_sm{1};
  std::atomic<int64_t> force_generic{0};          // 1 = always take the one-element-per-thread tier
  std::atomic<int64_t> pdl{1};                    // 1 = launch with programmatic stream serialization
  std::atomic<int64_t> wide{1};                   // 1 = 256-bit accesses where alignment allows
  std::atomic<int64_t> gather_rect_items{40000};  // padded (sequence, page, part, K|V) rectangles up to this size are walked as they are
  std::atomic<int64_t> write_prefetch_waves{2};   // leading write CTAs (in units of 8 per SM) that prefetch their rows into the L2
  std::atomic<int64_t> attn_min_items{0};         // decode attention: work items wanted before chunks stop halving (0 = built in)
  std::atomic<int64_t> attn_carry{1};             // decode attention: first loads of the next work item ahead of an item's epilogue (0 = off)
  std::atomic<int64_t> host_pair_kv{1};           // host-buffer gather: K and V run of a sequence as one 2-D copy where the outputs allow it (0 = two copies)
  std::atomic<int64_t> packed_fill_halves{1};     // packed write: prefetch the sector a lone half-sector store goes to (0 = off)
  std::atomic<int64_t> packed_lines_variant{0};   // packed write, whole-line kernel: 0 = 2 load rounds per thread, 6 CTAs per SM; 1 = 4 rounds, 4 CTAs
  std::atomic<int64_t> f8_tile_mult{8};           // fp8 wide write: bytes per CTA relative to the copy write
  std::atomic<int64_t> f8_unroll{1};              // fp8 wide write: 32-byte vectors of K and of V in flight per thread
  std::atomic<int64_t> packed_tile_tokens{32};    // tokens per CTA of the packed-page write
  std::atomic<int64_t> packed_tiles{1};           // 1 = transposing tile kernels for HND_PACKED pages where they apply
  std::atomic<int64_t> bulk_wait_us{1000000};     // a bulk-path wait on a copy is abandoned after this long
  std::atomic<int64_t> bulk_test_stall{0};        // test hook: pipe 0 of CTA 0 first waits on a barrier nothing completes
};
Options g_opt;
inline int64_t opt(const std::atomic<int64_t> &knob) { return knob.load(std::memory_order_relaxed); }
std::atomic<uint64_t> g_launches{0};

struct OptionName {
  const char *name;
  std::atomic<int64_t> Options::*field;
};
const OptionName kOptionNames[] = {
    {"write_vecs_per_cta", &Options::write_vecs_per_cta},
    {"write_unroll", &Options::write_unroll},
    {"gather_path", &Options::gather_path},
    {"gather_tile_bytes", &Options::gather_tile_bytes},
    {"gather_ctas_per_sm", &Options::gather_ctas_per_sm},
    {"write_prefetch_waves", &Options::write_prefetch_waves},
    {"gather_rect_items", &Options::gather_rect_items},
    {"gather_part_bytes", &Options::gather_part_bytes},
    {"bulk_stage_bytes", &Options::bulk_stage_bytes},
    {"bulk_stages", &Options::bulk_stages},
    {"bulk_pipes", &Options::bulk_pipes},
    {"bulk_lag", &Options::bulk_lag},
    {"bulk_ctas_per_sm", &Options::bulk_ctas_per_sm},
    {"force_generic", &Options::force_generic},
    {"pdl", &Options::pdl},
    {"wide", &Options::wide},
    {"attn_min_items", &Options::attn_min_items},
    {"attn_carry", &Options::attn_carry},
    {"host_pair_kv", &Options::host_pair_kv},
    {"packed_fill_halves", &Options::packed_fill_halves},
    {"packed_lines_variant", &Options::packed_lines_variant},
    {"f8_tile_mult", &Options::f8_tile_mult},
    {"f8_unroll", &Options::f8_unroll},
    {"packed_tile_tokens", &Options::packed_tile_tokens},
    {"packed_tiles", &Options::packed_tiles},
    {"bulk_wait_us", &Options::bulk_wait_us},
    {"bulk_test_stall", &Options::bulk_test_stall},
};

// Per-device facts, looked up once (never per launch).
struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
};
DeviceInfo g_dev[64];
std::atomic<int> g_dev_ready[64];

const DeviceInfo &device_info() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (g_dev_ready[dev].load(std::memory_order_acquire) == 0) {
    DeviceInfo info;
    cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (info.sm_count <= 0) info.sm_count = 148;
    g_dev[dev] = info;
    g_dev_ready[dev].store(1, std::memory_order_release);
  }
  return g_dev[dev];
}

// ------------------------------------------------------------------ geometry ----------

using kvx_detail::PageView;
using kvx_detail::ScaleView;
using kvx_detail::dtype_bytes;
using kvx_detail::make_page_view;
using kvx_detail::resolve_scale;

struct Geometry {
  int32_t num_blocks, block_size, heads, dim;
  int32_t elem;  // bytes per cache element
};

bool aligned(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }
int shift_of(int64_t v) {  // log2 for powers of two, -1 otherwise
  if (!is_pow2(v)) return -1;
  int s = 0;
  while ((int64_t{1} << s) < v) ++s;
  return s;
}

// `dim` is contiguous (d -> d*elem bytes) in this view?
bool dim_contiguous(const PageView &v, int64_t elem, int64_t dim) {
  if (v.pack == 1) return v.dhi == elem;
  return v.pack == dim && v.dlo == elem;
}

// Can this view be addressed with `vec`-byte vectors along dim?
bool view_vectorisable(const PageView &v, int64_t elem, int64_t dim, int64_t vec) {
  return dim_contiguous(v, elem, dim) && (dim * elem) % vec == 0 && aligned(v.base, vec) &&
         v.blk % vec == 0 && v.tok % vec == 0 && v.head % vec == 0 && v.blk >= 0 && v.tok >= 0 &&
         v.head >= 0;
}

// HND_PACKED pages whose pack group is one 16-byte vector (pack * elem == 16, the packing vLLM's
// and TGI's non-flash paged attention use) or 2^k of them (32, 64 ... bytes): the groups of one
// head are then `dhi` bytes apart instead of adjacent, and a token's groups pack * elem bytes
// apart.  *sub = k: vector w of a head lies at (w >> k) * dhi + (w & (2^k - 1)) * 16.
bool view_packed16(const PageView &v, int64_t elem, int64_t dim, int32_t *sub) {
  const int64_t u = v.pack * elem;
  *sub = 0;
  if (!(v.pack > 1 && v.pack != dim && u % 16 == 0 && is_pow2(u / 16) && v.dlo == elem && aligned(v.base, 16) &&
        v.blk % 16 == 0 && v.tok % 16 == 0 && v.tok >= u && v.head % 16 == 0 && v.dhi % 16 == 0 && v.blk >= 0 && v.head >= 0 && v.dhi >= 0))
    return false;
  *sub = shift_of(u / 16);
  return true;
}

// One packed page tensor as the tile kernels see it (device code reads it too).
struct PackedSide {
  int64_t dhi;      // bytes between consecutive pack groups of one head
  int32_t n_shift;  // log2(16 / u): 0 for 16-byte units ... 3 for 2-byte units
  int32_t runs;     // 32-byte units per group row (block_size * u / 32)
  int32_t runs_shift;
};

// HND_PACKED pages the transposing tile kernels take: pack groups of u = 2, 4, 8 or 16 bytes,
// the groups of consecutive tokens adjacent (tok == u), a group row (block_size * u bytes) made
// of whole 32-byte units, everything 32-byte aligned.  pack = 1 is the [blocks, heads, dim,
// block_size] tensor vLLM's and TGI's non-flash attention keep V in.
bool view_packed_tile(const PageView &v, int64_t elem, int64_t dim, int64_t block_size, PackedSide *out) {
  const int64_t u = v.pack * elem;
  if (u != 2 && u != 4 && u != 8 && u != 16) return false;
  if (v.pack == dim && dim > 1) return false;  // dim contiguous: an ordinary HND tensor
  if (v.pack > 1 && v.dlo != elem) return false;
  if (v.tok != u || (block_size * u) % 32 != 0 || v.dhi < block_size * u) return false;
  if (!aligned(v.base, 32) || v.blk % 32 != 0 || v.head % 32 != 0 || v.dhi % 32 != 0 || v.blk < 0 || v.head < 0)
    return false;
  out->dhi = v.dhi;
  out->n_shift = shift_of(16 / u);
  out->runs = static_cast<int32_t>(block_size * u / 32);
  out->runs_shift = shift_of(out->runs);
  return true;
}

// ------------------------------------------------------------------ device helpers ----

// Set to 1 when a bounded wait gives up (the bulk gather path is the only place that waits);
// the host reads and clears it with kvx_b200_device_error().
__device__ int g_device_error;

__device__ __forceinline__ uint4 load_stream(const void *p) {
  // Read-once data: bypass L1 allocation.
  uint4 r;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void store_stream(void *p, const uint4 &r) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.x), "r"(r.y), "r"(r.z),
               "r"(r.w)
               : "memory");
}

// 256-bit global accesses (sm_100): half the memory instructions of the 128-bit form for the
// same bytes; addresses must be 32-byte aligned.
struct Vec32 {
  uint32_t w[8];
};
__device__ __forceinline__ Vec32 load_stream32(const void *p) {
  Vec32 r;
  asm volatile("ld.global.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]),
                 "=r"(r.w[7])
               : "l"(p));
  return r;
}
__device__ __forceinline__ void store_stream32(void *p, const Vec32 &r) {
  asm volatile("st.global.cs.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.w[0]), "r"(r.w[1]),
               "r"(r.w[2]), "r"(r.w[3]), "r"(r.w[4]), "r"(r.w[5]), "r"(r.w[6]), "r"(r.w[7])
               : "memory");
}

// Programmatic dependent launch.  Every streaming kernel starts with pdl_prologue(): it lets
// the NEXT kernel in the stream begin scheduling its CTAs while this one is still running,
// then waits until everything that was enqueued BEFORE this kernel has completed and its
// writes are visible.  No global memory is touched before that wait, so stream order is kept;
// what is gained is the launch latency and CTA ramp-up between back-to-back per-layer calls
// (a no-op when the kernel was launched without the attribute).
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The two halves of pdl_prologue() for kernels that warm the L2 in between.  A prefetch
// consumes no value: the L2 is the point of coherence, so a line fetched early still shows
// what the previous kernel writes to it later, and stream order is kept as above.
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Byte offset of 16-byte vector w of a head whose pack groups (2^sub vectors each) are `step`
// bytes apart; step = 16, sub = 0 for a head that is contiguous.
__device__ __forceinline__ int64_t group_vec_offset(int w, int64_t step, int sub) {
  return static_cast<int64_t>(w >> sub) * step + ((w & ((1 << sub) - 1)) << 4);
}

// n / d and n % d for a runtime d with a known power-of-two shift (or -1).
__device__ __forceinline__ int div_by(int n, int d, int shift) {
  return shift >= 0 ? (n >> shift) : (n / d);
}

__device__ __forceinline__ void split_slot(int64_t slot, int32_t block_size, int bs_shift,
                                           int64_t *block, int64_t *off) {
  if (bs_shift >= 0) {
    *block = slot >> bs_shift;
    *off = slot & (block_size - 1);
  } else if ((slot >> 31) == 0) {  // fits 32 bits: cheap division
    const uint32_t s = static_cast<uint32_t>(slot);
    const uint32_t b = s / static_cast<uint32_t>(block_size);
    *block = b;
    *off = s - b * static_cast<uint32_t>(block_size);
  } else {
    *block = slot / block_size;
    *off = slot - *block * block_size;
  }
}

// ------------------------------------------------------------------ write: vector tier -

constexpr int kWriteThreads = 256;
constexpr int kMaxTokTile = 128;

struct WriteRowsParams {
  const char *key, *value;  // dense [T, row_bytes]
  char *k_base, *v_base;
  int64_t k_blk, k_tok, k_head;  // bytes
  int64_t v_blk, v_tok, v_head;
  int64_t k_vec, v_vec;  // bytes between consecutive pack groups of one head (16 unless packed)
  int32_t k_sub, v_sub;  // log2 of the 16-byte vectors per pack group (0 unless the groups are 32 bytes or more)
  int64_t k_pitch, v_pitch;  // bytes between consecutive token rows of key / value (row_bytes when dense)
  const void *slots;
  int64_t row_bytes;
  int32_t num_tokens, num_blocks, block_size, bs_shift;
  int32_t vpr, vpr_shift;  // 16-byte vectors per token row
  int32_t vps, vps_shift;  // 16-byte vectors per head segment
  int32_t tok_tile;        // tokens per CTA (<= kMaxTokTile)
  int32_t tile_shift;      // log2(tok_tile), used by the token-fastest order only
  int32_t early_ctas;      // CTAs that can be resident before the previous kernel has ended
};

// pdl_prologue() of the write kernels.  Between letting the next kernel in and waiting for the
// previous one, the leading CTAs of the grid ask for their slots and their dense key / value
// rows: CTAs that sit at the wait while the previous kernel drains then start from the L2, and
// in a launch no larger than that (a shard of the batch) the rows are on their way while the
// slots are still being turned into page offsets.  Further CTAs skip it: once the kernel runs
// at the memory's rate the extra requests only cost (padded rows are asked for too).
template <typename SlotT>
__device__ __forceinline__ void write_prologue(const WriteRowsParams &p, int64_t tok0, int ntok, bool pitched) {
  pdl_release();
  if (!pitched && static_cast<int>(blockIdx.x) < p.early_ctas) {
    const int tid = threadIdx.x;
    if (tid * 128 < ntok * static_cast<int>(sizeof(SlotT)))
      prefetch_l2(static_cast<const char *>(p.slots) + tok0 * sizeof(SlotT) + tid * 128);
    const int64_t bytes = ntok * p.row_bytes;
    for (int64_t off = static_cast<int64_t>(tid) * 128; off < bytes; off += kWriteThreads * 128) {
      prefetch_l2(p.key + tok0 * p.row_bytes + off);
      prefetch_l2(p.value + tok0 * p.row_bytes + off);
    }
  }
  pdl_wait();
}

// kSeg = false: every token row is one contiguous span in both page tensors.
// kSeg = true : a row is num_heads spans of head_dim elements (HND pages, or NHD pages whose
//               head stride is not head_dim), or, in HND_PACKED pages with 16-byte pack
//               groups, num_heads * head_dim / pack separate vectors (k_vec / v_vec apart).
// kTrans      : threads run over tokens fastest, vectors slowest (tok_tile is a power of two).
//               For packed pages the stores of neighbouring threads are then adjacent (the same
//               vector of consecutive slots) and it is the loads that are 16-byte pieces.
// kPitched    : token rows of key / value are k_pitch / v_pitch bytes apart (slices of a fused
//               projection output) instead of dense.
template <typename SlotT, bool kSeg, int kUnroll, bool kTrans = false, bool kPitched = false>
__global__ void __launch_bounds__(kWriteThreads) kvx_write_rows_kernel(const WriteRowsParams p) {
  __shared__ int64_t s_k[kMaxTokTile];
  __shared__ int64_t s_v[kMaxTokTile];
  const int tid = threadIdx.x;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * p.tok_tile;
  const int ntok = static_cast<int>(min(static_cast<int64_t>(p.tok_tile), p.num_tokens - tok0));
  write_prologue<SlotT>(p, tok0, ntok, kPitched);

  if (tid < ntok) {
    const int64_t slot = static_cast<int64_t>(static_cast<const SlotT *>(p.slots)[tok0 + tid]);
    int64_t ko = -1, vo = -1;
    if (slot >= 0) {  // negative = padding (reference: kernels/kvx_paged_kv.cu:137-140)
      int64_t b, o;
      split_slot(slot, p.block_size, p.bs_shift, &b, &o);
      if (b < p.num_blocks) {  // out-of-range block: skipped, not an error (:143-145)
        ko = b * p.k_blk + o * p.k_tok;
        vo = b * p.v_blk + o * p.v_tok;
      }
    }
    s_k[tid] = ko;
    s_v[tid] = vo;
  }
  __syncthreads();

  const char *ksrc = p.key + tok0 * (kPitched ? p.k_pitch : p.row_bytes);
  const char *vsrc = p.value + tok0 * (kPitched ? p.v_pitch : p.row_bytes);
  const int nvec = (kTrans ? p.tok_tile : ntok) * p.vpr;
  for (int f0 = tid; f0 < nvec; f0 += kWriteThreads * kUnroll) {
    uint4 kr[kUnroll], vr[kUnroll];
    int64_t kd[kUnroll], vd[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int f = f0 + u * kWriteThreads;
      kd[u] = -1;
      if (f < nvec) {
        const int tok = kTrans ? (f & (p.tok_tile - 1)) : div_by(f, p.vpr, p.vpr_shift);
        const int64_t ko = (!kTrans || tok < ntok) ? s_k[tok] : -1;
        if (ko >= 0) {
          const int v = kTrans ? (f >> p.tile_shift) : f - tok * p.vpr;
          if (kSeg) {
            const int h = div_by(v, p.vps, p.vps_shift);
            const int64_t w = v - h * p.vps;
            kd[u] = ko + h * p.k_head + group_vec_offset(w, p.k_vec, p.k_sub);
            vd[u] = s_v[tok] + h * p.v_head + group_vec_offset(w, p.v_vec, p.v_sub);
          } else {
            kd[u] = ko + static_cast<int64_t>(v) * 16;
            vd[u] = s_v[tok] + static_cast<int64_t>(v) * 16;
          }
          if (kPitched) {
            kr[u] = load_stream(ksrc + tok * p.k_pitch + static_cast<int64_t>(v) * 16);
            vr[u] = load_stream(vsrc + tok * p.v_pitch + static_cast<int64_t>(v) * 16);
          } else {
            const int64_t from = kTrans ? static_cast<int64_t>(tok) * p.vpr + v : f;
            kr[u] = load_stream(ksrc + from * 16);
            vr[u] = load_stream(vsrc + from * 16);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (kd[u] >= 0) {
        store_stream(p.k_base + kd[u], kr[u]);
        store_stream(p.v_base + vd[u], vr[u]);
      }
    }
  }
}

// ------------------------------------------------------------------ element converters -

struct F16 {
  uint16_t bits;
};
struct BF16 {
  uint16_t bits;
};
struct F32 {
  uint32_t bits;
};
struct F8 {
  uint8_t bits;
};

__device__ __forceinline__ float to_f32(F16 x) { return __half2float(__ushort_as_half(x.bits)); }
__device__ __forceinline__ float to_f32(BF16 x) {
  return __uint_as_float(static_cast<uint32_t>(x.bits) << 16);
}
__device__ __forceinline__ float to_f32(F32 x) { return __uint_as_float(x.bits); }

// Two f32 -> two E4M3 bytes with one rounding each (nearest even, saturating to +-448);
// `lo` lands in bits 0-7.  A NaN input yields 0x7F whatever its sign.
__device__ __forceinline__ uint32_t e4m3x2_from_f32(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  uint32_t q = r;
  if (lo != lo) q = (q & 0xFF00u) | 0x7Fu;
  if (hi != hi) q = (q & 0x00FFu) | 0x7F00u;
  return q;
}

// Quantise: one IEEE division, then one rounding to E4M3.
__device__ __forceinline__ uint32_t quant2(float lo, float hi, float scale) {
  return e4m3x2_from_f32(__fdiv_rn(lo, scale), __fdiv_rn(hi, scale));
}

// Division-free quantisation that is still bit-identical to the division.
// The reference result is e4m3(RN(x / s)).  RN(x / s) itself is rebuilt from the correctly
// rounded reciprocal r = RN(1 / s) with two residual corrections (Markstein): q0 = RN(x r) is
// within 2 ulp of x / s, q1 = RN(q0 + r (x - s q0)) is a faithful rounding, and one more step
// from a faithful start is the correctly rounded quotient.  The residuals are exact because
// they are formed by fused multiply-adds.  Five float-pipe operations replace a division that
// costs twice as many issue slots plus two trips through the conversion unit.
//   * -0 would come out as +0, so the sign of x is copied onto the result.
//   * +-inf, NaN and quotients beyond the f32 range turn into NaN inside the chain; a NaN
//     code (0x7F / 0xFF) anywhere in a vector's result sends it to the division route, which
//     handles them (a finite quotient never converts to the NaN code: the conversion saturates).
//   * a quotient too small for exact residuals is far below 2^-11 and rounds to zero anyway,
//     provided the scale is within 2^-60 .. 2^60; other scales take the division route.
__device__ __forceinline__ float fast_reciprocal(float s) {  // 0 = this scale must use the division
  const bool ok = (s >= 8.673617379884035e-19f) && (s <= 1.152921504606847e18f);  // 2^-60 .. 2^60; NaN fails
  return ok ? __frcp_rn(s) : 0.f;
}
__device__ __forceinline__ float quotient_rn(float x, float s, float r) {
  const float q0 = __fmul_rn(x, r);
  const float q1 = __fmaf_rn(__fmaf_rn(-s, q0, x), r, q0);
  const float q2 = __fmaf_rn(__fmaf_rn(-s, q1, x), r, q1);
  return __uint_as_float((__float_as_uint(q2) & 0x7FFFFFFFu) | (__float_as_uint(x) & 0x80000000u));
}
__device__ __forceinline__ uint32_t quant2_fast(float lo, float hi, float s, float r) {
  const float qlo = quotient_rn(lo, s, r), qhi = quotient_rn(hi, s, r);
  uint16_t c;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(c) : "f"(qhi), "f"(qlo));
  return c;
}
// The same without the sign copy: only x = -0 comes out with the wrong sign (+0); the caller
// repairs the signs of four results at once from the inputs' sign bytes.
__device__ __forceinline__ float quotient_rn_unsigned_zero(float x, float s, float r) {
  const float q0 = __fmul_rn(x, r);
  const float q1 = __fmaf_rn(__fmaf_rn(-s, q0, x), r, q0);
  return __fmaf_rn(__fmaf_rn(-s, q1, x), r, q1);
}
__device__ __forceinline__ uint32_t quant2_fast_unsigned_zero(float lo, float hi, float s, float r) {
  const float qlo = quotient_rn_unsigned_zero(lo, s, r), qhi = quotient_rn_unsigned_zero(hi, s, r);
  uint16_t c;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(c) : "f"(qhi), "f"(qlo));
  return c;
}

// The same for a pair of elements at once with the packed f32x2 arithmetic of sm_100 (one issue
// slot for two products or two fused multiply-adds; each half rounds exactly like the scalar
// instruction, denormals are kept): half the float-pipe instructions of the scalar chain.
// neg_s = {-s, -s}, r = {RN(1 / s), RN(1 / s)}.
__device__ __forceinline__ uint32_t quant2_packed_unsigned_zero(float2 x, float2 neg_s, float2 r) {
  const float2 q0 = __fmul2_rn(x, r);
  const float2 q1 = __ffma2_rn(__ffma2_rn(neg_s, q0, x), r, q0);
  const float2 q2 = __ffma2_rn(__ffma2_rn(neg_s, q1, x), r, q1);
  uint16_t c;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(c) : "f"(q2.y), "f"(q2.x));
  return c;
}

// Two E4M3 bytes (bits 0-15) -> two f32, exact.
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t q) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(q)));
  return __half22float2(*reinterpret_cast<__half2 *>(&h2));
}

// Round f32 to the IO element type (nearest even); NaN becomes the canonical quiet NaN.
__device__ __forceinline__ F16 from_f32(float z, F16) {
  return F16{__half_as_ushort(__float2half_rn(z))};
}
__device__ __forceinline__ BF16 from_f32(float z, BF16) {
  return BF16{__bfloat16_as_ushort(__float2bfloat16_rn(z))};
}
__device__ __forceinline__ F32 from_f32(float z, F32) {
  return F32{(z != z) ? 0x7FFFFFFFu : __float_as_uint(z)};
}

template <typename T>
struct ElemTraits;
template <>
struct ElemTraits<F16> {
  static constexpr int per_vec = 8;  // elements in 16 bytes
};
template <>
struct ElemTraits<BF16> {
  static constexpr int per_vec = 8;
};
template <>
struct ElemTraits<F32> {
  static constexpr int per_vec = 4;
};

// 16 bytes of IO elements -> per_vec E4M3 bytes (8 or 4), packed little-endian.
__device__ __forceinline__ void unpack_vec(const uint4 &x, float (&f)[8], BF16) {
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void unpack_vec(const uint4 &x, float (&f)[8], F16) {
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void unpack_vec(const uint4 &x, float (&f)[8], F32) {
  f[0] = __uint_as_float(x.x), f[1] = __uint_as_float(x.y);
  f[2] = __uint_as_float(x.z), f[3] = __uint_as_float(x.w);
  f[4] = f[5] = f[6] = f[7] = 0.f;
}

// The IEEE-division route for one vector.  Kept out of line on purpose: it runs for a few
// vectors in 10^4, and inlined it would be if-converted into the hot loop and issued (predicated
// off) for every vector.
template <typename IoT>
__device__ __noinline__ uint2 quant_vec_exact(uint4 x, float scale) {
  constexpr int kPairs = ElemTraits<IoT>::per_vec / 2;
  float f[8];
  unpack_vec(x, f, IoT{});
  uint32_t q[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int i = 0; i < kPairs; ++i) q[i] = quant2(f[2 * i], f[2 * i + 1], scale);
  return make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
}

// `r` = fast_reciprocal(scale), 0 when the scale rules the fast route out.
template <typename IoT>
__device__ __forceinline__ uint2 quant_vec(const uint4 &x, float scale, float r, IoT) {
  constexpr int kPairs = ElemTraits<IoT>::per_vec / 2;
  float f[8];
  unpack_vec(x, f, IoT{});
  uint32_t q[4] = {0u, 0u, 0u, 0u};
  uint2 out;
  if constexpr (ElemTraits<IoT>::per_vec == 8) {
    // 16-bit inputs: the sign of element i is the top bit of byte 2 i + 1 of the vector, so one
    // byte permute gathers four sign bytes and one logic operation puts them on four results
    // (instead of one sign copy per element inside the quotient).
    const float2 neg_s = make_float2(-scale, -scale), r2 = make_float2(r, r);
#pragma unroll
    for (int i = 0; i < kPairs; ++i) q[i] = quant2_packed_unsigned_zero(make_float2(f[2 * i], f[2 * i + 1]), neg_s, r2);
    const uint32_t lo = q[0] | (q[1] << 16), hi = q[2] | (q[3] << 16);
    out.x = (lo & 0x7F7F7F7Fu) | (__byte_perm(x.x, x.y, 0x7531) & 0x80808080u);
    out.y = (hi & 0x7F7F7F7Fu) | (__byte_perm(x.z, x.w, 0x7531) & 0x80808080u);
  } else {
#pragma unroll
    for (int i = 0; i < kPairs; ++i) q[i] = quant2_fast(f[2 * i], f[2 * i + 1], scale, r);
    out = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
  }
  // bytes equal to 0x7F after dropping the sign = NaN codes
  const uint32_t nan_bytes = __vcmpeq4(out.x & 0x7F7F7F7Fu, 0x7F7F7F7Fu) | __vcmpeq4(out.y & 0x7F7F7F7Fu, 0x7F7F7F7Fu);
  if (nan_bytes != 0u || r == 0.f)  // inf / NaN / out-of-range quotient somewhere, or an extreme scale
    return quant_vec_exact<IoT>(x, scale);
  return out;
}

// per_vec E4M3 bytes -> 16 bytes of IO elements: hardware e4m3x2 -> f16x2 (exact), widen to
// f32, one multiply, one rounding to the IO type.  (Building the f32 directly from the byte
// with integer operations was measured slower: it moves the work onto the integer pipe, which
// then becomes the limiter.)
__device__ __forceinline__ uint32_t pack2(float lo, float hi, BF16) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi, F16) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}
template <typename IoT>
__device__ __forceinline__ uint4 dequant_vec(uint2 q, float scale, IoT) {
  const uint32_t w[4] = {q.x & 0xFFFFu, q.x >> 16, q.y & 0xFFFFu, q.y >> 16};
  if constexpr (ElemTraits<IoT>::per_vec == 4) {
    const float2 a = e4m3x2_to_f32(w[0]), b = e4m3x2_to_f32(w[1]);
    return make_uint4(from_f32(a.x * scale, F32{}).bits, from_f32(a.y * scale, F32{}).bits,
                      from_f32(b.x * scale, F32{}).bits, from_f32(b.y * scale, F32{}).bits);
  } else {
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = e4m3x2_to_f32(w[i]);
      o[i] = pack2(f.x * scale, f.y * scale, IoT{});  // NaN packs as the canonical 0x7FFF
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------------ write: fp8 vector --

#ifndef KVX_F8_WRITE_UNROLL
#define KVX_F8_WRITE_UNROLL 2  // input vectors of K and of V in flight per thread
#endif
constexpr int kF8CachedHeads = 128;

struct WriteF8Params {
  WriteRowsParams w;  // vpr / vps count 16-byte INPUT vectors; k_*/v_* strides are cache bytes
  ScaleView ks, vs;
  int32_t dim;    // head_dim
  int32_t heads;  // num_kv_heads
};

// Same token tiling as kvx_write_rows_kernel; each 16-byte input vector (8 or 4 elements,
// all of one head) becomes 8 or 4 cache bytes.
// kPow2: vectors per row and per head are powers of two (shifts instead of divisions).
template <typename IoT, typename SlotT, int kUnroll, bool kPitched = false, bool kPow2 = false>
__global__ void __launch_bounds__(kWriteThreads) kvx_write_f8_kernel(const WriteF8Params q) {
  constexpr int kPer = ElemTraits<IoT>::per_vec;
  const WriteRowsParams &p = q.w;
  __shared__ int64_t s_k[kMaxTokTile];
  __shared__ int64_t s_v[kMaxTokTile];
  __shared__ float4 s_scale[kF8CachedHeads];  // per head: K scale, its fast_reciprocal, V scale, its fast_reciprocal
  const int tid = threadIdx.x;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * p.tok_tile;
  const int ntok = static_cast<int>(min(static_cast<int64_t>(p.tok_tile), p.num_tokens - tok0));
  write_prologue<SlotT>(p, tok0, ntok, kPitched);
  const bool cached = q.heads <= kF8CachedHeads;
  const int k_head32 = static_cast<int>(p.k_head), v_head32 = static_cast<int>(p.v_head);
  if (cached) {
    for (int h = tid; h < q.heads; h += kWriteThreads) {
      const float a = __ldg(q.ks.base + h * q.ks.stride), b = __ldg(q.vs.base + h * q.vs.stride);
      s_scale[h] = make_float4(a, fast_reciprocal(a), b, fast_reciprocal(b));
    }
  }
  if (tid < ntok) {
    const int64_t slot = static_cast<int64_t>(static_cast<const SlotT *>(p.slots)[tok0 + tid]);
    int64_t ko = -1, vo = -1;
    if (slot >= 0) {
      int64_t b, o;
      split_slot(slot, p.block_size, p.bs_shift, &b, &o);
      if (b < p.num_blocks) {
        ko = b * p.k_blk + o * p.k_tok;
        vo = b * p.v_blk + o * p.v_tok;
      }
    }
    s_k[tid] = ko;
    s_v[tid] = vo;
  }
  __syncthreads();

  const char *ksrc = p.key + tok0 * (kPitched ? p.k_pitch : p.row_bytes);
  const char *vsrc = p.value + tok0 * (kPitched ? p.v_pitch : p.row_bytes);
  const int nvec = ntok * p.vpr;
  for (int f0 = tid; f0 < nvec; f0 += kWriteThreads * kUnroll) {
    uint4 kr[kUnroll], vr[kUnroll];
    int64_t kd[kUnroll], vd[kUnroll];
    int hh[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int f = f0 + u * kWriteThreads;
      kd[u] = -1;
      if (f < nvec) {
        const int tok = kPow2 ? (f >> p.vpr_shift) : div_by(f, p.vpr, p.vpr_shift);
        const int64_t ko = s_k[tok];
        if (ko >= 0) {
          const int v = f - tok * p.vpr;
          const int h = kPow2 ? (v >> p.vps_shift) : div_by(v, p.vps, p.vps_shift);
          const int w = (v - h * p.vps) * kPer;  // cache bytes into the head
          hh[u] = h;
          // offsets inside a page fit 32 bits (the launcher checks the head pitch)
          kd[u] = ko + (h * k_head32 + w);
          vd[u] = s_v[tok] + (h * v_head32 + w);
          if (kPitched) {
            kr[u] = load_stream(ksrc + tok * p.k_pitch + static_cast<int64_t>(v) * 16);
            vr[u] = load_stream(vsrc + tok * p.v_pitch + static_cast<int64_t>(v) * 16);
          } else {
            kr[u] = load_stream(ksrc + static_cast<int64_t>(f) * 16);
            vr[u] = load_stream(vsrc + static_cast<int64_t>(f) * 16);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (kd[u] >= 0) {
        float sk, rk, sv, rv;
        if (cached) {
          const float4 sc = s_scale[hh[u]];
          sk = sc.x, rk = sc.y, sv = sc.z, rv = sc.w;
        } else {
          sk = __ldg(q.ks.base + hh[u] * q.ks.stride), sv = __ldg(q.vs.base + hh[u] * q.vs.stride);
          rk = fast_reciprocal(sk), rv = fast_reciprocal(sv);
        }
        const uint2 a = quant_vec(kr[u], sk, rk, IoT{});
        const uint2 b = quant_vec(vr[u], sv, rv, IoT{});
        if (kPer == 8) {
          *reinterpret_cast<uint2 *>(p.k_base + kd[u]) = a;
          *reinterpret_cast<uint2 *>(p.v_base + vd[u]) = b;
        } else {
          *reinterpret_cast<uint32_t *>(p.k_base + kd[u]) = a.x;
          *reinterpret_cast<uint32_t *>(p.v_base + vd[u]) = b.x;
        }
      }
    }
  }
}

// The common case of kvx_write_f8_kernel with 256-bit loads: 16-bit inputs, dense rows, vectors
// per row and per head powers of two, per-head constants in shared memory.  One thread turns 32
// bytes of K and 32 bytes of V (16 + 16 elements of one head) into two 16-byte stores, which
// halves the index arithmetic per element -- the kernel is bound by instruction issue.
// p.vpr / p.vps count 32-byte input vectors here.
template <typename IoT, typename SlotT, int kUnroll>
__global__ void __launch_bounds__(kWriteThreads) kvx_write_f8_wide_kernel(const WriteF8Params q) {
  const WriteRowsParams &p = q.w;
  __shared__ int64_t s_k[kMaxTokTile];
  __shared__ int64_t s_v[kMaxTokTile];
  __shared__ float4 s_scale[kF8CachedHeads];
  const int tid = threadIdx.x;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * p.tok_tile;
  const int ntok = static_cast<int>(min(static_cast<int64_t>(p.tok_tile), p.num_tokens - tok0));
  write_prologue<SlotT>(p, tok0, ntok, false);
  const int k_head32 = static_cast<int>(p.k_head), v_head32 = static_cast<int>(p.v_head);
  for (int h = tid; h < q.heads; h += kWriteThreads) {
    const float a = __ldg(q.ks.base + h * q.ks.stride), b = __ldg(q.vs.base + h * q.vs.stride);
    s_scale[h] = make_float4(a, fast_reciprocal(a), b, fast_reciprocal(b));
  }
  if (tid < ntok) {
    const int64_t slot = static_cast<int64_t>(static_cast<const SlotT *>(p.slots)[tok0 + tid]);
    int64_t ko = -1, vo = -1;
    if (slot >= 0) {
      int64_t b, o;
      split_slot(slot, p.block_size, p.bs_shift, &b, &o);
      if (b < p.num_blocks) {
        ko = b * p.k_blk + o * p.k_tok;
        vo = b * p.v_blk + o * p.v_tok;
      }
    }
    s_k[tid] = ko;
    s_v[tid] = vo;
  }
  __syncthreads();

  const char *ksrc = p.key + tok0 * p.row_bytes;
  const char *vsrc = p.value + tok0 * p.row_bytes;
  const int nvec = ntok * p.vpr;
  for (int f0 = tid; f0 < nvec; f0 += kWriteThreads * kUnroll) {
    Vec32 kr[kUnroll], vr[kUnroll];
    int64_t ko[kUnroll];
    // all loads of the round first, so that kUnroll x 64 bytes per thread are in flight
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int f = f0 + u * kWriteThreads;
      ko[u] = f < nvec ? s_k[f >> p.vpr_shift] : -1;
      if (ko[u] >= 0) {
        kr[u] = load_stream32(ksrc + static_cast<int64_t>(f) * 32);
        vr[u] = load_stream32(vsrc + static_cast<int64_t>(f) * 32);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (ko[u] < 0) continue;
      const int f = f0 + u * kWriteThreads;
      const int tok = f >> p.vpr_shift;
      const int v = f - (tok << p.vpr_shift);
      const int h = v >> p.vps_shift;
      const int w = (v - (h << p.vps_shift)) * 16;  // cache bytes into the head
      const float4 sc = s_scale[h];
      const uint2 a0 = quant_vec(make_uint4(kr[u].w[0], kr[u].w[1], kr[u].w[2], kr[u].w[3]), sc.x, sc.y, IoT{});
      const uint2 a1 = quant_vec(make_uint4(kr[u].w[4], kr[u].w[5], kr[u].w[6], kr[u].w[7]), sc.x, sc.y, IoT{});
      const uint2 b0 = quant_vec(make_uint4(vr[u].w[0], vr[u].w[1], vr[u].w[2], vr[u].w[3]), sc.z, sc.w, IoT{});
      const uint2 b1 = quant_vec(make_uint4(vr[u].w[4], vr[u].w[5], vr[u].w[6], vr[u].w[7]), sc.z, sc.w, IoT{});
      *reinterpret_cast<uint4 *>(p.k_base + ko[u] + (h * k_head32 + w)) = make_uint4(a0.x, a0.y, a1.x, a1.y);
      *reinterpret_cast<uint4 *>(p.v_base + s_v[tok] + (h * v_head32 + w)) = make_uint4(b0.x, b0.y, b1.x, b1.y);
    }
  }
}

// ------------------------------------------------------------------ generic tier ------

struct GenericParams {
  PageView k, v;  // byte strides
  Geometry g;
  ScaleView ks, vs;
};

template <typename T>
__device__ __forceinline__ T load_elem(const char *p) {
  return *reinterpret_cast<const T *>(p);
}

__device__ __forceinline__ int64_t page_byte_offset(const PageView &v, int64_t b, int64_t o, int64_t h,
                                                    int32_t d) {
  const int32_t hi = d / v.pack;
  return b * v.blk + o * v.tok + h * v.head + hi * v.dhi + (d - hi * v.pack) * v.dlo;
}

// Element conversion between IO type and cache type.  Same type = bit copy.
template <typename SrcT, typename DstT>
struct Convert {
  static __device__ __forceinline__ DstT apply(SrcT x, float) {
    DstT r;
    r.bits = x.bits;
    return r;
  }
};
template <typename SrcT>
struct Convert<SrcT, F8> {  // quantise
  static __device__ __forceinline__ F8 apply(SrcT x, float scale) {
    return F8{static_cast<uint8_t>(e4m3x2_from_f32(__fdiv_rn(to_f32(x), scale), 0.f) & 0xFFu)};
  }
};
// One (token, head, dim) element per thread, any layout / stride / alignment.
template <typename IoT, typename CacheT, typename SlotT>
__global__ void __launch_bounds__(256)
    kvx_write_generic_kernel(const IoT *key, const IoT *value, int64_t k_pitch, int64_t v_pitch, const void *slots,
                             int64_t num_tokens, const GenericParams p) {  // pitches in elements
  const int64_t hd = static_cast<int64_t>(p.g.heads) * p.g.dim;
  const int64_t total = num_tokens * hd;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / hd;
  const int32_t rem = static_cast<int32_t>(idx - t * hd);
  const int32_t h = rem / p.g.dim;
  const int32_t d = rem - h * p.g.dim;
  const int64_t slot = static_cast<int64_t>(static_cast<const SlotT *>(slots)[t]);
  if (slot < 0) return;
  const int64_t b = slot / p.g.block_size;
  const int64_t o = slot - b * p.g.block_size;
  if (b >= p.g.num_blocks) return;
  const float sk = p.ks.base ? __ldg(p.ks.base + h * p.ks.stride) : 1.f;
  const float sv = p.vs.base ? __ldg(p.vs.base + h * p.vs.stride) : 1.f;
  *reinterpret_cast<CacheT *>(p.k.base + page_byte_offset(p.k, b, o, h, d)) =
      Convert<IoT, CacheT>::apply(key[t * k_pitch + rem], sk);
  *reinterpret_cast<CacheT *>(p.v.base + page_byte_offset(p.v, b, o, h, d)) =
      Convert<IoT, CacheT>::apply(value[t * v_pitch + rem], sv);
}

struct GatherShape {
  const void *table, *lens;
  int64_t table_bytes;  // bytes of `table` the leading CTAs prefetch into the L2 (0 = none)
  int32_t seq_count, max_blocks, max_seq_len;
  // RAGGED tables: table[indptr[s] + tok] is the page of token `tok` of sequence s, for
  // tok < indptr[s + 1] - indptr[s] (one entry per cached token).
  const void *indptr;  // NULL = PACKED
  int32_t indptr64;    // indptr entries are 64-bit
  int64_t indices_count;  // entries of `table` (RAGGED): tokens whose entry would lie outside are skipped
  // KV_OFFSETS tables (KVX_SPEC.md:116-122, KV_CACHE_LAYOUTS.md:89-96): int32
  // [S, beam_width, 2, max_blocks]; entry [s][0][0][lb] names the K page and [s][0][1][lb] the V
  // page of logical block lb.  Bit 31 of an entry selects the secondary pool, the low 31 bits
  // count pool blocks: page = pool + offset * pool_block_bytes.
  const char *pool[2];  // primary, secondary (may be NULL); pool[0] == NULL = not KV_OFFSETS
  int64_t pool_block_bytes;
  int32_t beam_width;
  // Un-padded output (kvx_launch_gather_kv_varlen): token tok of sequence s goes to output row
  // out_indptr[s] + tok while that stays below out_indptr[s + 1] and below out_rows.
  const void *out_indptr;  // NULL = padded [S, max_seq_len, H, D] output
  int32_t out_indptr64;
  int64_t out_rows;
};

// First byte of the K (kv = 0) or V (kv = 1) page of logical block lb of sequence seq in a
// KV_OFFSETS table, or NULL when the entry is skipped: it names the secondary pool and there
// is none, or its offset is not below num_blocks (the bound holds for either pool).
__device__ __forceinline__ const char *offsets_page(const GatherShape &s, int32_t num_blocks, int32_t seq,
                                                    int32_t lb, int kv) {
  const int64_t at = ((static_cast<int64_t>(seq) * s.beam_width) * 2 + kv) * s.max_blocks + lb;
  const uint32_t e = static_cast<const uint32_t *>(s.table)[at];
  const char *base = s.pool[e >> 31];
  const uint32_t off = e & 0x7FFFFFFFu;
  if (base == nullptr || off >= static_cast<uint32_t>(num_blocks)) return nullptr;
  return base + static_cast<int64_t>(off) * s.pool_block_bytes;
}

__device__ __forceinline__ int64_t read_indptr(const GatherShape &s, int64_t i) {
  return s.indptr64 ? static_cast<const int64_t *>(s.indptr)[i]
                    : static_cast<int64_t>(static_cast<const int32_t *>(s.indptr)[i]);
}

template <typename IdxT>
__device__ __forceinline__ int64_t read_idx(const void *p, int64_t i) {
  return static_cast<int64_t>(static_cast<const IdxT *>(p)[i]);
}

// Where sequence `seq` lands in the output: its first row, and how many of its tokens may be
// written (seq_lens, max_seq_len and, for the un-padded form, the rows set aside for it).
struct OutSpan {
  int64_t first_row, tokens;
};

template <typename IdxT>
__device__ __forceinline__ OutSpan out_span(const GatherShape &s, int32_t seq) {
  const int64_t len = min(read_idx<IdxT>(s.lens, seq), static_cast<int64_t>(s.max_seq_len));
  if (s.out_indptr == nullptr) return OutSpan{static_cast<int64_t>(seq) * s.max_seq_len, len};
  const int64_t first = s.out_indptr64 ? static_cast<const int64_t *>(s.out_indptr)[seq]
                                       : static_cast<int64_t>(static_cast<const int32_t *>(s.out_indptr)[seq]);
  const int64_t next = s.out_indptr64 ? static_cast<const int64_t *>(s.out_indptr)[seq + 1]
                                      : static_cast<int64_t>(static_cast<const int32_t *>(s.out_indptr)[seq + 1]);
  if (first < 0) return OutSpan{0, 0};
  return OutSpan{first, min(len, min(next, s.out_rows) - first)};
}

// One output element per thread over the padded [S, Lmax, H, D] rectangle.
template <typename IoT, typename CacheT, typename IdxT, bool kDequant>
__global__ void __launch_bounds__(256)
    kvx_gather_generic_kernel(IoT *key_out, IoT *value_out, const GatherShape s, const GenericParams p) {
  const int64_t hd = static_cast<int64_t>(p.g.heads) * p.g.dim;
  const int64_t total = static_cast<int64_t>(s.seq_count) * s.max_seq_len * hd;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t row = idx / hd;
  const int32_t rem = static_cast<int32_t>(idx - row * hd);
  const int32_t h = rem / p.g.dim;
  const int32_t d = rem - h * p.g.dim;
  const int32_t seq = static_cast<int32_t>(row / s.max_seq_len);
  const int32_t tok = static_cast<int32_t>(row - static_cast<int64_t>(seq) * s.max_seq_len);
  const OutSpan span = out_span<IdxT>(s, seq);
  if (tok >= span.tokens) return;
  const int64_t out = (span.first_row + tok) * hd + rem;  // element index in the output tensors
  const int32_t lb = tok / p.g.block_size;
  const int64_t o = tok - static_cast<int64_t>(lb) * p.g.block_size;
  const char *kp, *vp;  // the element's address in its K / V page, NULL = skipped
  if (s.pool[0] != nullptr) {
    if (lb >= s.max_blocks) return;
    kp = offsets_page(s, p.g.num_blocks, seq, lb, 0);
    vp = offsets_page(s, p.g.num_blocks, seq, lb, 1);
    if (kp != nullptr) kp += page_byte_offset(p.k, 0, o, h, d);
    if (vp != nullptr) vp += page_byte_offset(p.v, 0, o, h, d);
  } else {
    int64_t b;
    if (s.indptr != nullptr) {
      const int64_t first = read_indptr(s, seq);
      if (tok >= read_indptr(s, seq + 1) - first) return;
      if (first < 0 || first + tok >= s.indices_count) return;  // damaged indptr: skipped, like a bad page id
      b = read_idx<IdxT>(s.table, first + tok);
    } else {
      if (lb >= s.max_blocks) return;
      b = read_idx<IdxT>(s.table, static_cast<int64_t>(seq) * s.max_blocks + lb);
    }
    if (b < 0 || b >= p.g.num_blocks) return;
    kp = p.k.base + page_byte_offset(p.k, b, o, h, d);
    vp = p.v.base + page_byte_offset(p.v, b, o, h, d);
  }
  if (kp != nullptr) {
    const CacheT q = load_elem<CacheT>(kp);
    if (kDequant) {
      key_out[out] = from_f32(e4m3x2_to_f32(q.bits).x * __ldg(p.ks.base + h * p.ks.stride), IoT{});
    } else {
      IoT a;
      a.bits = q.bits;
      key_out[out] = a;
    }
  }
  if (vp != nullptr) {
    const CacheT q = load_elem<CacheT>(vp);
    if (kDequant) {
      value_out[out] = from_f32(e4m3x2_to_f32(q.bits).x * __ldg(p.vs.base + h * p.vs.stride), IoT{});
    } else {
      IoT a;
      a.bits = q.bits;
      value_out[out] = a;
    }
  }
}

// ------------------------------------------------------------------ gather: vector tier -

constexpr int kGatherThreads = 256;
constexpr int kGatherWarps = kGatherThreads / 32;

struct GatherPagesParams {
  const char *k_base, *v_base;
  int64_t k_blk, k_tok, k_head;  // bytes
  int64_t v_blk, v_tok, v_head;
  int64_t k_vec, v_vec;  // bytes between consecutive pack groups of one head (16 unless packed)
  int32_t k_sub, v_sub;  // log2 of the 16-byte vectors per pack group
  char *key_out, *value_out;
  GatherShape s;
  int64_t out_row_bytes;  // bytes of one output token row
  int32_t num_blocks, block_size;
  int32_t vpr, vpr_shift;  // 16-byte OUTPUT vectors per token row
  int32_t vps, vps_shift;  // 16-byte output vectors per head segment
  int32_t part_vecs;       // output vectors one work item covers
  int32_t parts;           // work items per full page chunk
  int32_t use_prefix;      // 1: prefix[] in shared memory holds compacted page counts
  int32_t dim;             // head_dim (fp8 variant)
  ScaleView ks, vs;        // fp8 variant
};

// Pages sequence s really has: ceil(min(len, Lmax) / bs), clamped to the table width.
template <typename IdxT>
__device__ __forceinline__ int32_t pages_of(const GatherPagesParams &p, int32_t seq) {
  int64_t len = read_idx<IdxT>(p.s.lens, seq);
  if (len <= 0) return 0;
  if (len > p.s.max_seq_len) len = p.s.max_seq_len;
  const int64_t n = (len + p.block_size - 1) / p.block_size;
  return static_cast<int32_t>(min(n, static_cast<int64_t>(p.s.max_blocks)));
}

// Exclusive prefix sum of pages_of() over all sequences into prefix[0..S]; returns prefix[S].
template <typename IdxT>
__device__ int32_t build_page_prefix(const GatherPagesParams &p, int32_t *prefix, int32_t *warp_tot) {
  const int tid = threadIdx.x;
  const int S = p.s.seq_count;
  const int per = (S + kGatherThreads - 1) / kGatherThreads;
  const int begin = min(tid * per, S), end = min(begin + per, S);
  int32_t local = 0;
  for (int s = begin; s < end; ++s) local += pages_of<IdxT>(p, s);
  // inclusive scan of `local` across the CTA
  int32_t incl = local;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int32_t n = __shfl_up_sync(0xFFFFFFFFu, incl, d);
    if ((tid & 31) >= d) incl += n;
  }
  if ((tid & 31) == 31) warp_tot[tid >> 5] = incl;
  __syncthreads();
  int32_t base = 0;
  for (int w = 0; w < (tid >> 5); ++w) base += warp_tot[w];
  int32_t run = base + incl - local;  // exclusive prefix of this thread's first sequence
  for (int s = begin; s < end; ++s) {
    prefix[s] = run;
    run += pages_of<IdxT>(p, s);
  }
  if (tid == kGatherThreads - 1) prefix[S] = run;
  __syncthreads();
  return prefix[S];
}

struct ChunkRef {
  int32_t seq, lb;
};

// Compact chunk index -> (sequence, logical block): last s with prefix[s] <= c.
__device__ __forceinline__ ChunkRef find_chunk(const int32_t *prefix, int32_t S, int32_t c) {
  int lo = 0, hi = S;  // prefix[lo] <= c < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= c)
      lo = mid;
    else
      hi = mid;
  }
  return ChunkRef{lo, c - prefix[lo]};
}

// Everything a copy loop needs to know about one (sequence, page) chunk.
struct ChunkInfo {
  int64_t block;    // physical page, -1 = skip
  int32_t tokens;   // valid tokens in the chunk
  int64_t out_off;  // byte offset of the chunk's first row in the output tensors
};

template <typename IdxT, bool kOffsets = false>
__device__ __forceinline__ ChunkInfo resolve_chunk(const GatherPagesParams &p, int32_t seq, int32_t lb) {
  ChunkInfo c;
  c.block = -1;
  c.tokens = 0;
  c.out_off = 0;
  if (lb >= p.s.max_blocks) return c;
  // The table entry exists whatever the sequence's length: it is asked for together with the
  // length, not after it.
  int64_t b = 0;
  if (!kOffsets) b = read_idx<IdxT>(p.s.table, static_cast<int64_t>(seq) * p.s.max_blocks + lb);
  const OutSpan span = out_span<IdxT>(p.s, seq);
  const int64_t len = span.tokens;
  const int64_t first = static_cast<int64_t>(lb) * p.block_size;
  if (first >= len) return c;  // (reference: kernels/kvx_paged_kv.cu:247-253)
  if (b < 0 || b >= p.num_blocks) return c;  // negative id: skipped (:256-258); too large: skipped too
  c.block = b;  // with kOffsets 0: the K and the V page are looked up by the caller
  c.tokens = static_cast<int32_t>(min(len - first, static_cast<int64_t>(p.block_size)));
  c.out_off = (span.first_row + first) * p.out_row_bytes;
  return c;
}

// pdl_prologue() of the gather kernels: between letting the next kernel in and waiting for the
// previous one, the leading CTAs ask for the lengths and the block table, so that the lookups
// in front of the first data loads are answered by the L2.
template <typename IdxT>
__device__ __forceinline__ void gather_prologue(const GatherPagesParams &p) {
  pdl_release();
  if (p.s.table_bytes > 0) {
    const int64_t at = (static_cast<int64_t>(blockIdx.x) * kGatherThreads + threadIdx.x) * 128;
    if (at < p.s.table_bytes) prefetch_l2(static_cast<const char *>(p.s.table) + at);
    if (at < static_cast<int64_t>(p.s.seq_count) * static_cast<int64_t>(sizeof(IdxT)))
      prefetch_l2(static_cast<const char *>(p.s.lens) + at);
  }
  pdl_wait();
}

// Persistent CTAs; warp-granular work items (chunk, part, K|V).
//   kSeg = false : page rows are contiguous -> a chunk is one contiguous span on both sides.
//   kSeg = true  : per-head segments (HND pages or padded strides).
//   kOffsets     : KV_OFFSETS table; K and V pages are resolved separately (offsets_page).
template <typename IdxT, bool kSeg, int kUnroll, bool kOffsets = false>
__global__ void __launch_bounds__(kGatherThreads) kvx_gather_pages_kernel(const GatherPagesParams p) {
  gather_prologue<IdxT>(p);
  extern __shared__ int32_t s_prefix[];
  __shared__ int32_t s_warp_tot[kGatherWarps];
  int64_t chunks;
  if (p.use_prefix)
    chunks = build_page_prefix<IdxT>(p, s_prefix, s_warp_tot);
  else
    chunks = static_cast<int64_t>(p.s.seq_count) * p.s.max_blocks;

  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * kGatherWarps + (threadIdx.x >> 5);
  const int64_t warps = static_cast<int64_t>(gridDim.x) * kGatherWarps;
  const int64_t items = chunks * p.parts * 2;

  for (int64_t item = warp; item < items; item += warps) {
    const int kv = static_cast<int>(item & 1);
    const int64_t rest = item >> 1;
    const int64_t c = rest / p.parts;
    const int part = static_cast<int>(rest - c * p.parts);
    ChunkRef ref;
    if (p.use_prefix) {
      ref = find_chunk(s_prefix, p.s.seq_count, static_cast<int32_t>(c));
    } else {
      ref.seq = static_cast<int32_t>(c / p.s.max_blocks);
      ref.lb = static_cast<int32_t>(c - static_cast<int64_t>(ref.seq) * p.s.max_blocks);
    }
    const ChunkInfo ci = resolve_chunk<IdxT, kOffsets>(p, ref.seq, ref.lb);
    if (ci.block < 0) continue;
    const int nvec = ci.tokens * p.vpr;
    const int vbeg = part * p.part_vecs;
    const int vend = min(vbeg + p.part_vecs, nvec);
    const char *src;
    if (kOffsets) {
      src = offsets_page(p.s, p.num_blocks, ref.seq, ref.lb, kv);
      if (src == nullptr) continue;
    } else {
      src = kv ? p.v_base + ci.block * p.v_blk : p.k_base + ci.block * p.k_blk;
    }
    char *dst = (kv ? p.value_out : p.key_out) + ci.out_off;
    const int64_t tok_b = kv ? p.v_tok : p.k_tok;
    const int64_t head_b = kv ? p.v_head : p.k_head;
    const int64_t vec_b = kv ? p.v_vec : p.k_vec;
    const int vec_sub = kv ? p.v_sub : p.k_sub;

    for (int f0 = vbeg + lane; f0 < vend; f0 += 32 * kUnroll) {
      uint4 r[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < vend) {
          int64_t so;
          if (kSeg) {
            const int tok = div_by(f, p.vpr, p.vpr_shift);
            const int v = f - tok * p.vpr;
            const int h = div_by(v, p.vps, p.vps_shift);
            so = tok * tok_b + h * head_b + group_vec_offset(v - h * p.vps, vec_b, vec_sub);
          } else {
            so = static_cast<int64_t>(f) * 16;
          }
          r[u] = load_stream(src + so);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < vend) store_stream(dst + static_cast<int64_t>(f) * 16, r[u]);
      }
    }
  }
}

// Warp-granular gather of contiguous page chunks with 256-bit accesses: identical work
// decomposition to kvx_gather_pages_kernel<IdxT, false, *>, counted in 32-byte units.
// Needs 32-byte aligned bases, block strides and rows, and an even part_vecs.  kSeg: per-head
// segments in the pages (HND, padded pitches); token and head pitches and the segment length
// are then multiples of 32 bytes too.
template <typename IdxT, int kUnroll, bool kSeg = false>
__global__ void __launch_bounds__(kGatherThreads) kvx_gather_pages_wide_kernel(const GatherPagesParams p) {
  gather_prologue<IdxT>(p);
  extern __shared__ int32_t s_prefix[];
  __shared__ int32_t s_warp_tot[kGatherWarps];
  int64_t chunks;
  if (p.use_prefix)
    chunks = build_page_prefix<IdxT>(p, s_prefix, s_warp_tot);
  else
    chunks = static_cast<int64_t>(p.s.seq_count) * p.s.max_blocks;

  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * kGatherWarps + (threadIdx.x >> 5);
  const int64_t warps = static_cast<int64_t>(gridDim.x) * kGatherWarps;
  const int64_t items = chunks * p.parts * 2;
  const int part_units = p.part_vecs >> 1, row_units = p.vpr >> 1;

  for (int64_t item = warp; item < items; item += warps) {
    const int kv = static_cast<int>(item & 1);
    const int64_t rest = item >> 1;
    const int64_t c = rest / p.parts;
    const int part = static_cast<int>(rest - c * p.parts);
    ChunkRef ref;
    if (p.use_prefix) {
      ref = find_chunk(s_prefix, p.s.seq_count, static_cast<int32_t>(c));
    } else {
      ref.seq = static_cast<int32_t>(c / p.s.max_blocks);
      ref.lb = static_cast<int32_t>(c - static_cast<int64_t>(ref.seq) * p.s.max_blocks);
    }
    const ChunkInfo ci = resolve_chunk<IdxT>(p, ref.seq, ref.lb);
    if (ci.block < 0) continue;
    const int nunit = ci.tokens * row_units;
    const int ubeg = part * part_units;
    const int uend = min(ubeg + part_units, nunit);
    const char *src = kv ? p.v_base + ci.block * p.v_blk : p.k_base + ci.block * p.k_blk;
    char *dst = (kv ? p.value_out : p.key_out) + ci.out_off;
    const int64_t tok_b = kv ? p.v_tok : p.k_tok;
    const int64_t head_b = kv ? p.v_head : p.k_head;
    const int seg_units = p.vps >> 1;
    for (int f0 = ubeg + lane; f0 < uend; f0 += 32 * kUnroll) {
      Vec32 r[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < uend) {
          int64_t so;
          if (kSeg) {
            const int tok = div_by(f, row_units, p.vpr_shift >= 0 ? p.vpr_shift - 1 : -1);
            const int v = f - tok * row_units;
            const int h = div_by(v, seg_units, p.vps_shift >= 0 ? p.vps_shift - 1 : -1);
            so = tok * tok_b + h * head_b + static_cast<int64_t>(v - h * seg_units) * 32;
          } else {
            so = static_cast<int64_t>(f) * 32;
          }
          r[u] = load_stream32(src + so);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < uend) store_stream32(dst + static_cast<int64_t>(f) * 32, r[u]);
      }
    }
  }
}

// ------------------------------------------------------------------ packed pages -------
// HND_PACKED pages ([blocks, heads, dim / pack, block_size, pack]): inside a (page, head) tile
// the unit of `pack` elements (u = pack * elem bytes, 2 / 4 / 8 / 16) of token t and group g
// lies at g * dhi + t * u, while a dense token row holds its groups side by side -- the tile is
// the transpose, in units of u bytes, of the dense [token][group] block.  Both sides are
// accessed with full 16- or 32-byte vectors: a 16-byte page vector holds the unit of ONE group
// for n = 16 / u consecutive tokens, a 16-byte dense vector the units of n consecutive groups
// for ONE token, so n lanes that hold the page vectors of n consecutive groups exchange units
// (an n x n transposition of u-byte units by shuffles, log2 n steps) and end up with the dense
// vectors of n consecutive tokens, or the other way round for the write.  u = 16 needs no
// exchange at all.

// `upper` = this lane has the step's lane bit set; the partner is lane ^ d.
__device__ __forceinline__ void exchange_pairs(uint32_t (&w)[4], bool upper, int d) {  // units of 8 bytes
  uint32_t a = upper ? w[0] : w[2], b = upper ? w[1] : w[3];
  a = __shfl_xor_sync(0xFFFFFFFFu, a, d);
  b = __shfl_xor_sync(0xFFFFFFFFu, b, d);
  if (upper)
    w[0] = a, w[1] = b;
  else
    w[2] = a, w[3] = b;
}
__device__ __forceinline__ void exchange_words(uint32_t (&w)[4], bool upper, int d) {  // units of 4 bytes
  uint32_t a = upper ? w[0] : w[1], b = upper ? w[2] : w[3];
  a = __shfl_xor_sync(0xFFFFFFFFu, a, d);
  b = __shfl_xor_sync(0xFFFFFFFFu, b, d);
  if (upper)
    w[0] = a, w[2] = b;
  else
    w[1] = a, w[3] = b;
}
__device__ __forceinline__ void exchange_halves(uint32_t (&w)[4], bool upper) {  // units of 2 bytes, d = 1
  const uint32_t pick = upper ? 0x5410u : 0x7632u;  // the lower lane sends its odd units, the upper its even ones
  uint32_t a = __byte_perm(w[0], w[1], pick), b = __byte_perm(w[2], w[3], pick);
  a = __shfl_xor_sync(0xFFFFFFFFu, a, 1);
  b = __shfl_xor_sync(0xFFFFFFFFu, b, 1);
  if (upper) {
    w[0] = __byte_perm(a, w[0], 0x7610u), w[1] = __byte_perm(a, w[1], 0x7632u);
    w[2] = __byte_perm(b, w[2], 0x7610u), w[3] = __byte_perm(b, w[3], 0x7632u);
  } else {
    w[0] = __byte_perm(w[0], a, 0x5410u), w[1] = __byte_perm(w[1], a, 0x7610u);
    w[2] = __byte_perm(w[2], b, 0x5410u), w[3] = __byte_perm(w[3], b, 0x7610u);
  }
}

// Lane i of each aligned group of kN lanes holds the vector [x(i,0) .. x(i,kN-1)] of kN units;
// afterwards it holds [x(0,i) .. x(kN-1,i)].  Every lane of the warp must take part.
template <int kN>
__device__ __forceinline__ void transpose_units(uint32_t (&w)[4], int lane) {
  if constexpr (kN == 2) {
    exchange_pairs(w, lane & 1, 1);
  } else if constexpr (kN == 4) {
    exchange_pairs(w, lane & 2, 2);
    exchange_words(w, lane & 1, 1);
  } else if constexpr (kN == 8) {
    exchange_pairs(w, lane & 4, 4);
    exchange_words(w, lane & 2, 2);
    exchange_halves(w, lane & 1);
  }
}

// A piece (up to kUnroll * 32 of the 32-byte units) of one (page, head) tile, page -> dense rows.
// Lane slot j covers group g = (q / runs) * kN + j % kN and tokens [a * 2 kN, (a + 1) * 2 kN) with
// q = j / kN, a = q % runs: the kN lanes of a group share a and hold consecutive groups.
template <int kN, int kUnroll>
__device__ __forceinline__ void gather_packed_piece(const char *src, char *dst, int64_t out_row_bytes,
                                                    const PackedSide &side, int first_slot, int slots, int tokens,
                                                    int lane) {
  Vec32 x[kUnroll];
  int tok_a[kUnroll], vec[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const int j = first_slot + u * 32 + lane;
    const int q = j / kN, i = j & (kN - 1);
    const int gb = div_by(q, side.runs, side.runs_shift);
    const int a = q - gb * side.runs;
    tok_a[u] = j < slots ? a * 2 * kN + i : tokens;  // >= tokens: nothing to store
    vec[u] = gb;
    if (j < slots && a * 2 * kN < tokens) {
      x[u] = load_stream32(src + static_cast<int64_t>(gb * kN + i) * side.dhi + a * 32);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) x[u].w[k] = 0u;
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    uint32_t lo[4] = {x[u].w[0], x[u].w[1], x[u].w[2], x[u].w[3]};
    uint32_t hi[4] = {x[u].w[4], x[u].w[5], x[u].w[6], x[u].w[7]};
    transpose_units<kN>(lo, lane);
    transpose_units<kN>(hi, lane);
    char *row = dst + static_cast<int64_t>(tok_a[u]) * out_row_bytes + vec[u] * 16;
    if (tok_a[u] < tokens) store_stream(row, make_uint4(lo[0], lo[1], lo[2], lo[3]));
    if (tok_a[u] + kN < tokens) store_stream(row + kN * out_row_bytes, make_uint4(hi[0], hi[1], hi[2], hi[3]));
  }
}

// 16-byte units (kN = 1), whole 128-byte lines on both sides and whole token rows per warp.  One
// item = 8 consecutive tokens (4 token pairs = one 128-byte line of every group row) of one page,
// all heads: the warp reads, head by head, 8 group rows x 128 bytes per instruction (a lane takes
// 32 bytes of group 8 gh + lane / 4 at token pair 4 ah + lane % 4) and writes 4 token rows x 128
// bytes with each of its two store instructions, so that the 8 output rows, which are contiguous,
// are filled by this one warp.  Needs runs % 4 == 0 and a multiple of 8 groups per head.
// With few heads (a shard of them) such an item is too little to keep a warp's loads in flight
// between two table lookups, so an item then spans 2^span_shift neighbouring lines of the group
// rows (octets of tokens), walked fastest: a group row gives up 2^span_shift x 128 contiguous bytes.
template <int kUnroll>
__device__ __forceinline__ void gather_packed16_rows(const char *src, int64_t head_bytes, char *dst,
                                                     int64_t out_row_bytes, int64_t head_out_bytes,
                                                     const PackedSide &side, int ah0, int span_shift, int g_blocks,
                                                     int steps, int tokens, int lane) {
  const int g_lo = lane >> 2;
  if (8 * ah0 >= tokens) return;  // warp-uniform: none of the item's tokens exists
  const int total = steps << span_shift, span_mask = (1 << span_shift) - 1;
  for (int t0 = 0; t0 < total; t0 += kUnroll) {  // a step = 8 groups of one head, for one octet of tokens
    Vec32 x[kUnroll];
    int at[kUnroll], first[kUnroll];  // byte offset inside a token row; the lane's first token (-1: nothing)
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int t = t0 + u, st = t >> span_shift;
      const int a = (ah0 + (t & span_mask)) * 4 + (lane & 3);
      const int h = st / g_blocks, gh = st - h * g_blocks;
      const int g = gh * 8 + g_lo;
      at[u] = static_cast<int>(h * head_out_bytes) + g * 16;
      first[u] = t < total && 2 * a < tokens ? 2 * a : -1;
      if (first[u] >= 0) x[u] = load_stream32(src + h * head_bytes + static_cast<int64_t>(g) * side.dhi + a * 32);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (first[u] < 0) continue;
      char *row = dst + static_cast<int64_t>(first[u]) * out_row_bytes + at[u];
      store_stream(row, make_uint4(x[u].w[0], x[u].w[1], x[u].w[2], x[u].w[3]));
      if (first[u] + 1 < tokens) store_stream(row + out_row_bytes, make_uint4(x[u].w[4], x[u].w[5], x[u].w[6], x[u].w[7]));
    }
  }
}

// 2-byte units (kN = 8: a [dims, tokens] tile of 16-bit elements, the V tensor of the paged
// attention caches) with whole token rows per warp.  One item = the 16 tokens of one 32-byte unit
// of the group rows, all heads.  A lane reads two group rows (dims d and d + 32 of a block of 64
// dims), 8 lanes transpose 8 dims x 8 tokens twice each, and one more exchange between the lanes
// i and i ^ 4 puts the two blocks of 32 dims side by side, so that every store instruction
// writes 4 token rows x 128 bytes (64 dims) instead of 8 rows x 64 bytes.
template <int kPairs>
__device__ __forceinline__ void gather_packed2_rows(const char *src, int64_t head_bytes, char *dst,
                                                    int64_t out_row_bytes, int64_t head_out_bytes,
                                                    const PackedSide &side, int a, int blocks, int steps,
                                                    int tokens, int lane) {
  const int i = lane & 7, q = lane >> 3;
  const int t0 = a * 16;
  if (t0 >= tokens) return;  // warp-uniform
  const bool low = i < 4;
  char *row = dst + static_cast<int64_t>(t0 + (i & 3)) * out_row_bytes + (low ? 0 : 64) + q * 16;
  for (int s0 = 0; s0 < steps; s0 += kPairs) {  // a step = 64 dims of one head
    Vec32 x[kPairs], y[kPairs];
    int at[kPairs];
#pragma unroll
    for (int u = 0; u < kPairs; ++u) {
      const int s = s0 + u;
      const int h = s / blocks, b64 = s - h * blocks;
      at[u] = s < steps ? static_cast<int>(h * head_out_bytes) + b64 * 128 : -1;
      if (s < steps) {
        const char *from = src + h * head_bytes + static_cast<int64_t>(b64 * 64 + q * 8 + i) * side.dhi + a * 32;
        x[u] = load_stream32(from);
        y[u] = load_stream32(from + 32 * side.dhi);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) x[u].w[k] = y[u].w[k] = 0u;
      }
    }
#pragma unroll
    for (int u = 0; u < kPairs; ++u) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {  // tokens t0 .. t0 + 7, then t0 + 8 .. t0 + 15
        uint32_t a0[4] = {x[u].w[4 * half], x[u].w[4 * half + 1], x[u].w[4 * half + 2], x[u].w[4 * half + 3]};
        uint32_t a1[4] = {y[u].w[4 * half], y[u].w[4 * half + 1], y[u].w[4 * half + 2], y[u].w[4 * half + 3]};
        transpose_units<8>(a0, lane);  // lane i: token i of the half, dims 8 q .. 8 q + 7 of the first 32
        transpose_units<8>(a1, lane);  // ... of the second 32
        uint32_t first[4], second[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, low ? a1[k] : a0[k], 4);
          first[k] = low ? a0[k] : got;    // token i & 3:     lanes 0-3 their first 32 dims, lanes 4-7 the partner's second 32
          second[k] = low ? got : a1[k];   // token 4 + i & 3: lanes 0-3 the partner's first 32, lanes 4-7 their second 32
        }
        if (at[u] < 0) continue;
        const int tok = t0 + 8 * half + (i & 3);
        char *to = row + static_cast<int64_t>(8 * half) * out_row_bytes + at[u];
        if (tok < tokens) store_stream(to, make_uint4(first[0], first[1], first[2], first[3]));
        if (tok + 4 < tokens) store_stream(to + 4 * out_row_bytes, make_uint4(second[0], second[1], second[2], second[3]));
      }
    }
  }
}

struct GatherPackedParams {
  GatherPagesParams g;  // parts = heads * pieces per head; k_vec / v_vec unused
  PackedSide k, v;
  int32_t slots;   // 32-byte units of one (page, head) tile: block_size * head_dim * elem / 32
  int32_t pieces;  // work items per head
  int32_t rows;    // 1: 16-byte units, items of 8 token rows (gather_packed16_rows); then
                   // g.parts = 128-byte lines per group row and pieces = 8-group blocks per head.
                   // 2: 2-byte units, items of 16 token rows (gather_packed2_rows); then g.parts =
                   // 32-byte units per group row and pieces = 64-dim blocks per head
  int32_t span_shift;  // rows == 1: an item spans 2^span_shift lines of the group rows (g.parts counts items)
  int32_t only;    // -1: K and V; 0: K only; 1: V only (K and V of different kinds take a launch each)
  int64_t head_out_bytes;  // head_dim * elem
};

// Gather from packed pages: same work list as kvx_gather_pages_kernel (compacted (sequence,
// page) chunks, warp-granular items), an item being one piece of one head's tile of K or of V.
template <typename IdxT, int kUnroll, int kRows>
__global__ void __launch_bounds__(kGatherThreads) kvx_gather_packed_kernel(const GatherPackedParams pp) {
  const GatherPagesParams &p = pp.g;
  gather_prologue<IdxT>(p);
  extern __shared__ int32_t s_prefix[];
  __shared__ int32_t s_warp_tot[kGatherWarps];
  int64_t chunks;
  if (p.use_prefix)
    chunks = build_page_prefix<IdxT>(p, s_prefix, s_warp_tot);
  else
    chunks = static_cast<int64_t>(p.s.seq_count) * p.s.max_blocks;

  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * kGatherWarps + (threadIdx.x >> 5);
  const int64_t warps = static_cast<int64_t>(gridDim.x) * kGatherWarps;
  const int64_t items = chunks * p.parts * (pp.only < 0 ? 2 : 1);

  for (int64_t item = warp; item < items; item += warps) {
    const int kv = pp.only < 0 ? static_cast<int>(item & 1) : pp.only;
    const int64_t rest = pp.only < 0 ? (item >> 1) : item;
    const int64_t c = rest / p.parts;
    const int part = static_cast<int>(rest - c * p.parts);
    ChunkRef ref;
    if (p.use_prefix) {
      ref = find_chunk(s_prefix, p.s.seq_count, static_cast<int32_t>(c));
    } else {
      ref.seq = static_cast<int32_t>(c / p.s.max_blocks);
      ref.lb = static_cast<int32_t>(c - static_cast<int64_t>(ref.seq) * p.s.max_blocks);
    }
    const ChunkInfo ci = resolve_chunk<IdxT>(p, ref.seq, ref.lb);
    if (ci.block < 0) continue;  // warp-uniform: every lane stays for the shuffles below
    if constexpr (kRows == 1) {
      gather_packed16_rows<kUnroll>(kv ? p.v_base + ci.block * p.v_blk : p.k_base + ci.block * p.k_blk,
                                    kv ? p.v_head : p.k_head, (kv ? p.value_out : p.key_out) + ci.out_off,
                                    p.out_row_bytes, pp.head_out_bytes, kv ? pp.v : pp.k, part << pp.span_shift,
                                    pp.span_shift, pp.pieces, pp.pieces * (p.vpr / p.vps), ci.tokens, lane);
      continue;
    }
    if constexpr (kRows == 2) {
      gather_packed2_rows<2>(kv ? p.v_base + ci.block * p.v_blk : p.k_base + ci.block * p.k_blk,
                             kv ? p.v_head : p.k_head, (kv ? p.value_out : p.key_out) + ci.out_off, p.out_row_bytes,
                             pp.head_out_bytes, kv ? pp.v : pp.k, part, pp.pieces, pp.pieces * (p.vpr / p.vps),
                             ci.tokens, lane);
      continue;
    }
    const int h = part / pp.pieces;
    const int first_slot = (part - h * pp.pieces) * (32 * kUnroll);
    const char *src = (kv ? p.v_base + ci.block * p.v_blk + h * p.v_head : p.k_base + ci.block * p.k_blk + h * p.k_head);
    char *dst = (kv ? p.value_out : p.key_out) + ci.out_off + h * pp.head_out_bytes;
    const PackedSide &side = kv ? pp.v : pp.k;
    switch (side.n_shift) {
      case 0: gather_packed_piece<1, kUnroll>(src, dst, p.out_row_bytes, side, first_slot, pp.slots, ci.tokens, lane); break;
      case 1: gather_packed_piece<2, kUnroll>(src, dst, p.out_row_bytes, side, first_slot, pp.slots, ci.tokens, lane); break;
      case 2: gather_packed_piece<4, kUnroll>(src, dst, p.out_row_bytes, side, first_slot, pp.slots, ci.tokens, lane); break;
      default: gather_packed_piece<8, kUnroll>(src, dst, p.out_row_bytes, side, first_slot, pp.slots, ci.tokens, lane); break;
    }
  }
}

// ---- write into packed pages ----------------------------------------------------------
// Tokens arrive in any order and with holes (padding), but a page vector needs the units of
// n = 16 / u consecutive slots.  So the tile's tokens are first cut into FRAGMENTS: maximal
// runs of consecutive tokens whose slots are consecutive inside one aligned window of
// W = 2 n = 32 / u slots (the slots of one 32-byte unit of a group row).  A fragment belongs to
// the CTA that holds its first token, which reads up to W - 1 tokens past its tile's end to
// complete it; a tile's leading tokens that continue a fragment begun in the previous tile are
// left to that CTA.  Fragments never overlap, so every valid token is written exactly once.
// A fragment that fills its window is stored as one 32-byte unit per group, one that fills an
// aligned half as a 16-byte vector, anything else unit by unit.
constexpr int kPackedTile = 128;             // most tokens per CTA
constexpr int kPackedSlots = kPackedTile + 17;  // + the token before the tile + up to W - 1 = 15 after it

struct WritePackedParams {
  const char *key, *value;  // dense (or pitched) [T, heads * dim] rows
  int64_t k_pitch, v_pitch;
  char *k_base, *v_base;
  int64_t k_blk, k_head, v_blk, v_head;
  PackedSide k, v;
  const void *slots;
  int32_t num_tokens, num_blocks, block_size, bs_shift;
  int32_t vpr;             // 16-byte vectors per dense token row
  int32_t vph, vph_shift;  // ... per head
  int32_t tok_tile;        // power of two <= kPackedTile
  int32_t k_lines, v_lines;  // 1: that tensor (16-byte units) through write_packed16_lines
  int32_t fill_halves;       // whole-line routine: prefetch the sector that a lone 16-byte store goes to
};

// Stores the units of `w` (positions 0 .. kN-1 of a half window) whose bit is set in `mask`.
template <int kN>
__device__ __forceinline__ void store_units(char *dst, const uint32_t (&w)[4], uint32_t mask) {
  if constexpr (kN == 1) {
    if (mask & 1u) store_stream(dst, make_uint4(w[0], w[1], w[2], w[3]));
  } else if constexpr (kN == 2) {
    if (mask & 1u) *reinterpret_cast<uint2 *>(dst) = make_uint2(w[0], w[1]);
    if (mask & 2u) *reinterpret_cast<uint2 *>(dst + 8) = make_uint2(w[2], w[3]);
  } else if constexpr (kN == 4) {
    // aligned pairs of units go out as one 8-byte store
#pragma unroll
    for (int k = 0; k < 4; k += 2) {
      const uint32_t m = (mask >> k) & 3u;
      if (m == 3u)
        *reinterpret_cast<uint2 *>(dst + 4 * k) = make_uint2(w[k], w[k + 1]);
      else if (m & 1u)
        *reinterpret_cast<uint32_t *>(dst + 4 * k) = w[k];
      else if (m & 2u)
        *reinterpret_cast<uint32_t *>(dst + 4 * k + 4) = w[k + 1];
    }
  } else {
    // aligned runs of four and of two units go out as 8- and 4-byte stores (a half window with
    // one hole: three stores, not seven)
#pragma unroll
    for (int q = 0; q < 2; ++q) {  // units 4 q .. 4 q + 3 = words 2 q, 2 q + 1
      const uint32_t m = (mask >> (4 * q)) & 0xFu;
      if (m == 0xFu) {
        *reinterpret_cast<uint2 *>(dst + 8 * q) = make_uint2(w[2 * q], w[2 * q + 1]);
        continue;
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {  // units 4 q + 2 j, + 1 = word 2 q + j
        const uint32_t mm = (m >> (2 * j)) & 3u;
        const uint32_t word = w[2 * q + j];
        char *at = dst + 8 * q + 4 * j;
        if (mm == 3u)
          *reinterpret_cast<uint32_t *>(at) = word;
        else if (mm & 1u)
          *reinterpret_cast<uint16_t *>(at) = static_cast<uint16_t>(word);
        else if (mm & 2u)
          *reinterpret_cast<uint16_t *>(at + 2) = static_cast<uint16_t>(word >> 16);
      }
    }
  }
}

// One tensor (K or V) of one token tile.  s_slot[1 + p] is the slot of tile token p (or -1),
// for p = -1 .. tok_tile + 2 kN - 2.
template <int kN>
__device__ __forceinline__ void write_packed_tensor(const WritePackedParams &p, const char *rows, int64_t pitch,
                                                    char *base, int64_t blk, int64_t head, const PackedSide &side,
                                                    const int64_t *s_slot, int32_t *s_frag, int64_t *s_win,
                                                    int *s_count, int ntok) {
  constexpr int kW = 2 * kN;
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid == 0) *s_count = 0;
  __syncthreads();
  if (tid < ntok) {
    const int64_t sl = s_slot[1 + tid];
    const int64_t before = s_slot[tid];
    const int pos0 = static_cast<int>(sl & (kW - 1));
    const bool continues = sl >= 0 && before >= 0 && sl == before + 1 && pos0 != 0;
    if (sl >= 0 && !continues) {
      int len = 1;
      while (pos0 + len < kW && s_slot[1 + tid + len] == sl + len) ++len;
      const int at = atomicAdd(s_count, 1);
      s_frag[at] = tid | (pos0 << 8) | (len << 16);
      int64_t b, o;
      split_slot(sl - pos0, p.block_size, p.bs_shift, &b, &o);
      s_win[at] = b * blk + o * (16 / kN);  // the window's first unit (group 0 of head 0)
    }
  }
  __syncthreads();
  const int nfrag = *s_count;
  const int i = lane & (kN - 1);
  const int groups = 32 / kN;  // (fragment, dense vector) pairs one warp instruction covers
  const int total = nfrag * p.vpr;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * p.tok_tile;
  // Every lane of a warp runs the same number of rounds (the exchanges need all 32 lanes); a
  // round takes kRound (fragment, vector) pairs per lane group, all loads first.
  constexpr int kRound = 4;
  const int warp_stride = (kWriteThreads / 32) * groups;
  for (int e0 = (tid >> 5) * groups; e0 < total; e0 += warp_stride * kRound) {
    uint32_t lo[kRound][4], hi[kRound][4];
    int at[kRound];           // fragment, or -1
    int vec[kRound];
    uint32_t window[kRound];  // slots of the window the fragment fills
#pragma unroll
    for (int r = 0; r < kRound; ++r) {
      const int e = e0 + r * warp_stride + lane / kN;
      const bool live = e < total;
      int frag = 0, v = 0;
      if (live) {
        frag = e / p.vpr;
        v = e - frag * p.vpr;
      }
      const int32_t info = live ? s_frag[frag] : 0;
      const int first = info & 0xFF, pos0 = (info >> 8) & 0xFF, len = live ? (info >> 16) : 0;
      at[r] = live ? frag : -1;
      vec[r] = v;
      window[r] = ((1u << len) - 1u) << pos0;
      // window position i (lower half) and kN + i (upper half) -> token of the fragment, if any
      const int ra = i - pos0, rb = kN + i - pos0;
      const char *from = rows + (tok0 + first) * pitch + static_cast<int64_t>(v) * 16;
      uint4 x = make_uint4(0u, 0u, 0u, 0u), y = make_uint4(0u, 0u, 0u, 0u);
      if (ra >= 0 && ra < len) x = load_stream(from + ra * pitch);
      if (rb >= 0 && rb < len) y = load_stream(from + rb * pitch);
      lo[r][0] = x.x, lo[r][1] = x.y, lo[r][2] = x.z, lo[r][3] = x.w;
      hi[r][0] = y.x, hi[r][1] = y.y, hi[r][2] = y.z, hi[r][3] = y.w;
    }
#pragma unroll
    for (int r = 0; r < kRound; ++r) {
      transpose_units<kN>(lo[r], lane);
      transpose_units<kN>(hi[r], lane);
      if (at[r] < 0) continue;
      const int h = div_by(vec[r], p.vph, p.vph_shift);
      const int gb = vec[r] - h * p.vph;
      char *dst = base + s_win[at[r]] + h * head + static_cast<int64_t>(gb * kN + i) * side.dhi;
      const uint32_t half = (1u << kN) - 1u;
      const uint32_t ma = window[r] & half, mb = (window[r] >> kN) & half;
      if (ma == half && mb == half) {
        Vec32 y;
        y.w[0] = lo[r][0], y.w[1] = lo[r][1], y.w[2] = lo[r][2], y.w[3] = lo[r][3];
        y.w[4] = hi[r][0], y.w[5] = hi[r][1], y.w[6] = hi[r][2], y.w[7] = hi[r][3];
        store_stream32(dst, y);
      } else {
        if (ma == half)
          store_stream(dst, make_uint4(lo[r][0], lo[r][1], lo[r][2], lo[r][3]));
        else if (ma)
          store_units<kN>(dst, lo[r], ma);
        if (mb == half)
          store_stream(dst + 16, make_uint4(hi[r][0], hi[r][1], hi[r][2], hi[r][3]));
        else if (mb)
          store_units<kN>(dst + 16, hi[r], mb);
      }
    }
  }
}

// K and V both in 16-byte units with whole 128-byte lines on both sides (the mirror of
// gather_packed16_rows).  The window is the 8 slots of one line of a group row.  Here the tile's
// tokens are not cut into fragments but sorted into WINDOWS: a table says, for every window the
// tile touches, which token of the tile (if any) goes to each of its 8 slots.  Holes in the
// slots (padding) then cost nothing but the lanes they leave idle, where every hole used to
// start a new fragment and with it another pass of a warp over all group rows: with 10 % of
// the slots padded the tile has 1.5 times the fragments of a tile without holes, and the
// kernel, which keeps the load-store path 87 % busy without them, slowed down by as much.
// Windows end at the tile's borders (no tile depends on what its neighbour does), and tokens
// that lie far apart but share a window simply get a window entry each.
//
// Building the table: a valid token LEADS a window unless the nearest valid token among the 7
// before it lies in the same window.  Every valid token walks back to its leader (over holes and
// over members of its own window) and enters itself at its slot's position in the leader's table
// row, which is the row with the leader's own number in the tile (rows are cleared while the
// slots are loaded); leaders also add themselves to the list of windows.  One barrier.
// Work items are then (window, block of 8 groups): a lane takes slot pair a = lane % 4 of the
// window and group 8 gh + lane / 4, each of its two loads reads 4 token rows x 128 bytes per
// warp instruction and its 32-byte store fills, with the three other pairs, one line of each
// of 8 group rows.  Needs a multiple of 8 groups per head and block sizes that are multiples of 8.
// (A tokens-fastest route for tiles without a hole is 1-2 % faster in a short burst and 1-2 %
// slower once the device sits at its power limit, which back-to-back packed writes reach --
// about 950 W -- so there is one route.)
struct PackedWindows {
  int64_t *k_at, *v_at;  // [windows] byte offset of the window's first unit in the K / V pool (group 0, head 0)
  int32_t *leader;       // [windows] the leading token of the window = its row in `token`
  int16_t *token;        // [tokens][8] for a leader: the token of the tile at each slot of its window, -1 = none
  int *count;
};

// (the caller has cleared `token` and *count and put a barrier behind that and the slots)
__device__ __forceinline__ void build_packed_windows(const WritePackedParams &p, const int64_t *s_slot, const PackedWindows &w,
                                                     int ntok) {
  for (int t = threadIdx.x; t < ntok; t += kWriteThreads) {
    const int64_t sl = s_slot[1 + t];
    if (sl < 0) continue;
    int lead = t;
    for (;;) {  // does the nearest valid token among the 7 before `lead` share the window?
      int j = lead - 1;
      while (j >= 0 && j >= lead - 7 && s_slot[1 + j] < 0) --j;
      if (j < 0 || j < lead - 7 || (s_slot[1 + j] >> 3) != (sl >> 3)) break;
      lead = j;
    }
    w.token[8 * lead + static_cast<int>(sl & 7)] = static_cast<int16_t>(t);
    if (lead == t) {
      const int at = atomicAdd(w.count, 1);
      int64_t b, o;
      split_slot(sl & ~int64_t{7}, p.block_size, p.bs_shift, &b, &o);
      w.leader[at] = t;
      w.k_at[at] = b * p.k_blk + o * 16;
      w.v_at[at] = b * p.v_blk + o * 16;
    }
  }
}

template <int kRound>
__device__ __forceinline__ void write_packed16_windows(const WritePackedParams &p, const char *rows, int64_t pitch,
                                                       char *base, int64_t head, const PackedSide &side,
                                                       const int64_t *s_at, const int32_t *s_leader,
                                                       const int16_t *s_token, int windows) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int a = lane & 3, g_lo = lane >> 2;
  const int blocks_per_row = p.vpr >> 3;  // 8-group blocks of one token row (all heads)
  const int blocks_per_head = p.vph >> 3;
  const int total = windows * blocks_per_row;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * p.tok_tile;
  for (int e0 = tid >> 5; e0 < total; e0 += (kWriteThreads / 32) * kRound) {
    uint4 x[kRound], y[kRound];
    int64_t to[kRound];
    uint32_t have[kRound];  // bit 0: the pair's first slot gets a token, bit 1: its second
#pragma unroll
    for (int r = 0; r < kRound; ++r) {
      const int e = e0 + r * (kWriteThreads / 32);
      have[r] = 0u;
      if (e >= total) continue;
      const int win = e / blocks_per_row, blk8 = e - win * blocks_per_row;
      const uint32_t pair = *reinterpret_cast<const uint32_t *>(s_token + 8 * s_leader[win] + 2 * a);
      const int ta = static_cast<int16_t>(pair & 0xFFFFu), tb = static_cast<int16_t>(pair >> 16);
      const int h = blk8 / blocks_per_head, gh = blk8 - h * blocks_per_head;
      const char *from = rows + tok0 * pitch + static_cast<int64_t>(blk8 * 8 + g_lo) * 16;
      if (ta >= 0) x[r] = load_stream(from + ta * pitch), have[r] |= 1u;
      if (tb >= 0) y[r] = load_stream(from + tb * pitch), have[r] |= 2u;
      to[r] = s_at[win] + h * head + static_cast<int64_t>(gh * 8 + g_lo) * side.dhi + a * 32;
      // Half a sector (the pair's other slot gets nothing from this tile): ask for the sector
      // now, so that the 16 bytes meet it in the L2 and it leaves as a whole sector, instead of
      // the memory completing it with a read-modify-write of its own when it is evicted.
      if (p.fill_halves && (have[r] == 1u || have[r] == 2u)) prefetch_l2(base + to[r]);
    }
#pragma unroll
    for (int r = 0; r < kRound; ++r) {
      if (have[r] == 3u) {
        Vec32 v;
        v.w[0] = x[r].x, v.w[1] = x[r].y, v.w[2] = x[r].z, v.w[3] = x[r].w;
        v.w[4] = y[r].x, v.w[5] = y[r].y, v.w[6] = y[r].z, v.w[7] = y[r].w;
        store_stream32(base + to[r], v);
      } else if (have[r] == 1u) {
        store_stream(base + to[r], x[r]);
      } else if (have[r] == 2u) {
        store_stream(base + to[r] + 16, y[r]);
      }
    }
  }
}

// Slots of the tile's tokens, of the token before it and of up to 16 after it (-1: padding, or
// beyond the pool, which is skipped like padding): s_slot[1 + t] for token t of the tile.
template <typename SlotT>
__device__ __forceinline__ void load_tile_slots(const WritePackedParams &p, int64_t tok0, int64_t *s_slot) {
  const int tid = threadIdx.x;
  if (tid < p.tok_tile + 17) {
    const int64_t t = tok0 - 1 + tid;
    int64_t sl = -1;
    if (t >= 0 && t < p.num_tokens) {
      sl = static_cast<int64_t>(static_cast<const SlotT *>(p.slots)[t]);
      if (sl >= 0) {
        int64_t b, o;
        split_slot(sl, p.block_size, p.bs_shift, &b, &o);
        if (b >= p.num_blocks) sl = -1;
      }
    }
    s_slot[tid] = sl < 0 ? -1 : sl;
  }
}

// K and V both in 16-byte units, whole lines: one window table serves both tensors.
template <typename SlotT, int kRound, int kMinCtas>
__global__ void __launch_bounds__(kWriteThreads, kMinCtas) kvx_write_packed_lines_kernel(const WritePackedParams p) {
  __shared__ int64_t s_slot[kPackedSlots];
  __shared__ int64_t s_win[kPackedTile];
  __shared__ int64_t s_win_v[kPackedTile];
  __shared__ __align__(16) int16_t s_token[kPackedTile * 8];
  __shared__ int32_t s_leader[kPackedTile];
  __shared__ int s_count;
  pdl_prologue();
  const int tid = threadIdx.x;
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * p.tok_tile;
  const int ntok = static_cast<int>(min(static_cast<int64_t>(p.tok_tile), p.num_tokens - tok0));
  load_tile_slots<SlotT>(p, tok0, s_slot);
  for (int t = tid; t < ntok; t += kWriteThreads)
    *reinterpret_cast<uint4 *>(s_token + 8 * t) = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
  if (tid == 0) s_count = 0;
  __syncthreads();
  const PackedWindows w{s_win, s_win_v, s_leader, s_token, &s_count};
  build_packed_windows(p, s_slot, w, ntok);
  __syncthreads();
  const int windows = s_count;
  write_packed16_windows<kRound>(p, p.key, p.k_pitch, p.k_base, p.k_head, p.k, s_win, s_leader, s_token, windows);
  write_packed16_windows<kRound>(p, p.value, p.v_pitch, p.v_base, p.v_head, p.v, s_win_v, s_leader, s_token, windows);
}

template <typename SlotT>
__global__ void __launch_bounds__(kWriteThreads) kvx_write_packed_kernel(const WritePackedParams p) {
  __shared__ int64_t s_slot[kPackedSlots];
  __shared__ int64_t s_win[kPackedTile];
  __shared__ int32_t s_frag[kPackedTile];
  __shared__ int s_count;
  pdl_prologue();
  const int64_t tok0 = static_cast<int64_t>(blockIdx.x) * p.tok_tile;
  const int ntok = static_cast<int>(min(static_cast<int64_t>(p.tok_tile), p.num_tokens - tok0));
  load_tile_slots<SlotT>(p, tok0, s_slot);
  // (both tensor routines begin with a barrier)
#define KVX_PACKED_TENSOR(N, rows, pitch, base, blk, head, side) \
  write_packed_tensor<N>(p, rows, pitch, base, blk, head, side, s_slot, s_frag, s_win, &s_count, ntok)
  {
    switch (p.k.n_shift) {
      case 0: KVX_PACKED_TENSOR(1, p.key, p.k_pitch, p.k_base, p.k_blk, p.k_head, p.k); break;
      case 1: KVX_PACKED_TENSOR(2, p.key, p.k_pitch, p.k_base, p.k_blk, p.k_head, p.k); break;
      case 2: KVX_PACKED_TENSOR(4, p.key, p.k_pitch, p.k_base, p.k_blk, p.k_head, p.k); break;
      default: KVX_PACKED_TENSOR(8, p.key, p.k_pitch, p.k_base, p.k_blk, p.k_head, p.k); break;
    }
  }
  __syncthreads();  // the fragment list is rebuilt for V (its window may differ)
  {
    switch (p.v.n_shift) {
      case 0: KVX_PACKED_TENSOR(1, p.value, p.v_pitch, p.v_base, p.v_blk, p.v_head, p.v); break;
      case 1: KVX_PACKED_TENSOR(2, p.value, p.v_pitch, p.v_base, p.v_blk, p.v_head, p.v); break;
      case 2: KVX_PACKED_TENSOR(4, p.value, p.v_pitch, p.v_base, p.v_blk, p.v_head, p.v); break;
      default: KVX_PACKED_TENSOR(8, p.value, p.v_pitch, p.v_base, p.v_blk, p.v_head, p.v); break;
    }
  }
#undef KVX_PACKED_TENSOR
}

// CTA-granular variant: one work item = one part of a page chunk, K AND V, moved by the
// whole CTA with kUnroll K loads + kUnroll V loads in flight per thread before the first
// store (the same shape as one tile of the write kernel).  The next item's page id is
// resolved before the current item is copied, so the lens -> table -> page dependency chain
// never sits in front of the data loads.
template <typename IdxT, bool kSeg, int kUnroll>
__global__ void __launch_bounds__(kGatherThreads, 4) kvx_gather_tiles_kernel(const GatherPagesParams p) {
  gather_prologue<IdxT>(p);
  extern __shared__ int32_t s_prefix[];
  __shared__ int32_t s_warp_tot[kGatherWarps];
  int64_t chunks;
  if (p.use_prefix)
    chunks = build_page_prefix<IdxT>(p, s_prefix, s_warp_tot);
  else
    chunks = static_cast<int64_t>(p.s.seq_count) * p.s.max_blocks;
  const int tid = threadIdx.x;
  const int64_t items = chunks * p.parts;

  auto resolve_item = [&](int64_t item, int *part) {
    const int64_t c = item / p.parts;
    *part = static_cast<int>(item - c * p.parts);
    ChunkRef ref;
    if (p.use_prefix) {
      ref = find_chunk(s_prefix, p.s.seq_count, static_cast<int32_t>(c));
    } else {
      ref.seq = static_cast<int32_t>(c / p.s.max_blocks);
      ref.lb = static_cast<int32_t>(c - static_cast<int64_t>(ref.seq) * p.s.max_blocks);
    }
    return resolve_chunk<IdxT>(p, ref.seq, ref.lb);
  };

  int64_t item = blockIdx.x;
  if (item >= items) return;
  int part = 0;
  ChunkInfo cur = resolve_item(item, &part);
  while (true) {
    const int64_t next = item + gridDim.x;
    int next_part = 0;
    ChunkInfo nxt;
    nxt.block = -1, nxt.tokens = 0, nxt.out_off = 0;
    if (next < items) nxt = resolve_item(next, &next_part);

    if (cur.block >= 0) {
      const int nvec = cur.tokens * p.vpr;
      const int vbeg = part * p.part_vecs;
      const int vend = min(vbeg + p.part_vecs, nvec);
      const char *ksrc = p.k_base + cur.block * p.k_blk;
      const char *vsrc = p.v_base + cur.block * p.v_blk;
      char *kdst = p.key_out + cur.out_off;
      char *vdst = p.value_out + cur.out_off;
      for (int f0 = vbeg + tid; f0 < vend; f0 += kGatherThreads * kUnroll) {
        uint4 kr[kUnroll], vr[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int f = f0 + u * kGatherThreads;
          if (f < vend) {
            int64_t ko, vo;
            if (kSeg) {
              const int tok = div_by(f, p.vpr, p.vpr_shift);
              const int v = f - tok * p.vpr;
              const int h = div_by(v, p.vps, p.vps_shift);
              const int64_t w = static_cast<int64_t>(v - h * p.vps) * 16;
              ko = tok * p.k_tok + h * p.k_head + w;
              vo = tok * p.v_tok + h * p.v_head + w;
            } else {
              ko = vo = static_cast<int64_t>(f) * 16;
            }
            kr[u] = load_stream(ksrc + ko);
            vr[u] = load_stream(vsrc + vo);
          }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int f = f0 + u * kGatherThreads;
          if (f < vend) {
            store_stream(kdst + static_cast<int64_t>(f) * 16, kr[u]);
            store_stream(vdst + static_cast<int64_t>(f) * 16, vr[u]);
          }
        }
      }
    }
    if (next >= items) break;
    item = next, part = next_part, cur = nxt;
  }
}

// RAGGED block tables (one page id per cached token).  CTA = a tile of consecutive tokens of
// one sequence: the first threads resolve each token's page row into a source byte offset in
// shared memory, then all threads stream the tile's 16-byte vectors into the (contiguous)
// output rows -- the write kernel's shape with the indirection on the source side.
constexpr int kRaggedTile = 64;
template <typename IdxT, int kUnroll>
__global__ void __launch_bounds__(kGatherThreads) kvx_gather_ragged_kernel(const GatherPagesParams p) {
  pdl_prologue();
  __shared__ int64_t s_k[kRaggedTile];
  __shared__ int64_t s_v[kRaggedTile];
  const int tid = threadIdx.x;
  const int seq = blockIdx.y;
  const int t0 = blockIdx.x * p.part_vecs;  // part_vecs = tokens per CTA here
  const OutSpan span = out_span<IdxT>(p.s, seq);
  const int64_t first = read_indptr(p.s, seq);
  const int64_t len = min(span.tokens, read_indptr(p.s, seq + 1) - first);
  if (t0 >= len) return;
  const int ntok = static_cast<int>(min(static_cast<int64_t>(p.part_vecs), len - t0));
  if (tid < ntok) {
    const int tok = t0 + tid;
    // an entry outside the index array (damaged indptr) is skipped, like a bad page id
    const bool inside = first >= 0 && first + tok < p.s.indices_count;
    const int64_t b = inside ? read_idx<IdxT>(p.s.table, first + tok) : -1;
    int64_t ko = -1, vo = -1;
    if (b >= 0 && b < p.num_blocks) {
      const int64_t o = tok % p.block_size;
      ko = b * p.k_blk + o * p.k_tok;
      vo = b * p.v_blk + o * p.v_tok;
    }
    s_k[tid] = ko;
    s_v[tid] = vo;
  }
  __syncthreads();
  const int64_t out_off = (span.first_row + t0) * p.out_row_bytes;
  char *kdst = p.key_out + out_off;
  char *vdst = p.value_out + out_off;
  const int nvec = ntok * p.vpr;
  for (int f0 = tid; f0 < nvec; f0 += kGatherThreads * kUnroll) {
    uint4 kr[kUnroll], vr[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int f = f0 + u * kGatherThreads;
      live[u] = false;
      if (f < nvec) {
        const int tok = div_by(f, p.vpr, p.vpr_shift);
        const int64_t ko = s_k[tok];
        if (ko >= 0) {
          const int v = f - tok * p.vpr;
          const int h = div_by(v, p.vps, p.vps_shift);
          const int64_t w = static_cast<int64_t>(v - h * p.vps) * 16;
          kr[u] = load_stream(p.k_base + ko + h * p.k_head + w);
          vr[u] = load_stream(p.v_base + s_v[tok] + h * p.v_head + w);
          live[u] = true;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int f = f0 + u * kGatherThreads;
      if (live[u]) {
        store_stream(kdst + static_cast<int64_t>(f) * 16, kr[u]);
        store_stream(vdst + static_cast<int64_t>(f) * 16, vr[u]);
      }
    }
  }
}

// Dequantising gather: same decomposition; each 16-byte OUTPUT vector (8 or 4 elements of
// one head) is produced from 8 or 4 cache bytes.
template <typename IoT, typename IdxT, int kUnroll, bool kOffsets = false>
__global__ void __launch_bounds__(kGatherThreads) kvx_gather_f8_kernel(const GatherPagesParams p) {
  gather_prologue<IdxT>(p);
  constexpr int kPer = ElemTraits<IoT>::per_vec;
  extern __shared__ int32_t s_prefix[];
  __shared__ int32_t s_warp_tot[kGatherWarps];
  int64_t chunks;
  if (p.use_prefix)
    chunks = build_page_prefix<IdxT>(p, s_prefix, s_warp_tot);
  else
    chunks = static_cast<int64_t>(p.s.seq_count) * p.s.max_blocks;

  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * kGatherWarps + (threadIdx.x >> 5);
  const int64_t warps = static_cast<int64_t>(gridDim.x) * kGatherWarps;
  const int64_t items = chunks * p.parts * 2;

  for (int64_t item = warp; item < items; item += warps) {
    const int kv = static_cast<int>(item & 1);
    const int64_t rest = item >> 1;
    const int64_t c = rest / p.parts;
    const int part = static_cast<int>(rest - c * p.parts);
    ChunkRef ref;
    if (p.use_prefix) {
      ref = find_chunk(s_prefix, p.s.seq_count, static_cast<int32_t>(c));
    } else {
      ref.seq = static_cast<int32_t>(c / p.s.max_blocks);
      ref.lb = static_cast<int32_t>(c - static_cast<int64_t>(ref.seq) * p.s.max_blocks);
    }
    const ChunkInfo ci = resolve_chunk<IdxT, kOffsets>(p, ref.seq, ref.lb);
    if (ci.block < 0) continue;
    const int nvec = ci.tokens * p.vpr;
    const int vbeg = part * p.part_vecs;
    const int vend = min(vbeg + p.part_vecs, nvec);
    const char *src;
    if (kOffsets) {
      src = offsets_page(p.s, p.num_blocks, ref.seq, ref.lb, kv);
      if (src == nullptr) continue;
    } else {
      src = kv ? p.v_base + ci.block * p.v_blk : p.k_base + ci.block * p.k_blk;
    }
    char *dst = (kv ? p.value_out : p.key_out) + ci.out_off;
    const int64_t tok_b = kv ? p.v_tok : p.k_tok;
    const int64_t head_b = kv ? p.v_head : p.k_head;
    const ScaleView sc = kv ? p.vs : p.ks;

    for (int f0 = vbeg + lane; f0 < vend; f0 += 32 * kUnroll) {
      uint2 r[kUnroll];
      int hh[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < vend) {
          const int tok = div_by(f, p.vpr, p.vpr_shift);
          const int v = f - tok * p.vpr;
          const int h = div_by(v, p.vps, p.vps_shift);
          const char *a = src + tok * tok_b + h * head_b + static_cast<int64_t>(v - h * p.vps) * kPer;
          hh[u] = h;
          if (kPer == 8)
            r[u] = *reinterpret_cast<const uint2 *>(a);
          else
            r[u] = make_uint2(*reinterpret_cast<const uint32_t *>(a), 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < vend) {
          const float scale = __ldg(sc.base + hh[u] * sc.stride);
          store_stream(dst + static_cast<int64_t>(f) * 16, dequant_vec(r[u], scale, IoT{}));
        }
      }
    }
  }
}

// The dequantising gather with 256-bit stores: 16-bit outputs whose head rows are whole 32-byte
// vectors.  A lane turns 16 cache bytes (16 elements of one head) into one 32-byte store: half
// the memory instructions and half the index arithmetic per element of the kernel above.
// part_vecs, vpr and vps still count 16-byte output vectors (all even here).
template <typename IoT, typename IdxT, int kUnroll>
__global__ void __launch_bounds__(kGatherThreads) kvx_gather_f8_wide_kernel(const GatherPagesParams p) {
  gather_prologue<IdxT>(p);
  extern __shared__ int32_t s_prefix[];
  __shared__ int32_t s_warp_tot[kGatherWarps];
  int64_t chunks;
  if (p.use_prefix)
    chunks = build_page_prefix<IdxT>(p, s_prefix, s_warp_tot);
  else
    chunks = static_cast<int64_t>(p.s.seq_count) * p.s.max_blocks;

  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * kGatherWarps + (threadIdx.x >> 5);
  const int64_t warps = static_cast<int64_t>(gridDim.x) * kGatherWarps;
  const int64_t items = chunks * p.parts * 2;
  const int part_units = p.part_vecs >> 1, row_units = p.vpr >> 1, seg_units = p.vps >> 1;
  const int row_shift = p.vpr_shift >= 0 ? p.vpr_shift - 1 : -1, seg_shift = p.vps_shift >= 0 ? p.vps_shift - 1 : -1;

  for (int64_t item = warp; item < items; item += warps) {
    const int kv = static_cast<int>(item & 1);
    const int64_t rest = item >> 1;
    const int64_t c = rest / p.parts;
    const int part = static_cast<int>(rest - c * p.parts);
    ChunkRef ref;
    if (p.use_prefix) {
      ref = find_chunk(s_prefix, p.s.seq_count, static_cast<int32_t>(c));
    } else {
      ref.seq = static_cast<int32_t>(c / p.s.max_blocks);
      ref.lb = static_cast<int32_t>(c - static_cast<int64_t>(ref.seq) * p.s.max_blocks);
    }
    const ChunkInfo ci = resolve_chunk<IdxT>(p, ref.seq, ref.lb);
    if (ci.block < 0) continue;
    const int nunit = ci.tokens * row_units;
    const int ubeg = part * part_units;
    const int uend = min(ubeg + part_units, nunit);
    const char *src = kv ? p.v_base + ci.block * p.v_blk : p.k_base + ci.block * p.k_blk;
    char *dst = (kv ? p.value_out : p.key_out) + ci.out_off;
    const int64_t tok_b = kv ? p.v_tok : p.k_tok;
    const int64_t head_b = kv ? p.v_head : p.k_head;
    const ScaleView sc = kv ? p.vs : p.ks;

    for (int f0 = ubeg + lane; f0 < uend; f0 += 32 * kUnroll) {
      uint4 r[kUnroll];
      int hh[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < uend) {
          const int tok = div_by(f, row_units, row_shift);
          const int v = f - tok * row_units;
          const int h = div_by(v, seg_units, seg_shift);
          hh[u] = h;
          r[u] = *reinterpret_cast<const uint4 *>(src + tok * tok_b + h * head_b + static_cast<int64_t>(v - h * seg_units) * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int f = f0 + u * 32;
        if (f < uend) {
          const float scale = __ldg(sc.base + hh[u] * sc.stride);
          const uint4 lo = dequant_vec(make_uint2(r[u].x, r[u].y), scale, IoT{});
          const uint4 hi = dequant_vec(make_uint2(r[u].z, r[u].w), scale, IoT{});
          Vec32 out;
          out.w[0] = lo.x, out.w[1] = lo.y, out.w[2] = lo.z, out.w[3] = lo.w;
          out.w[4] = hi.x, out.w[5] = hi.y, out.w[6] = hi.z, out.w[7] = hi.w;
          store_stream32(dst + static_cast<int64_t>(f) * 32, out);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ gather: bulk tier --
// cp.async.bulk staging of contiguous page chunks: global -> shared (completion on an
// mbarrier) -> global (bulk group).  One elected thread ("pipe") owns a ring of stages and
// walks its share of the work items; the copy engine moves the bytes.

constexpr int kBulkMaxPipes = 8;
constexpr int kBulkMaxStages = 8;

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Wait for the phase with the given parity, for at most limit_ns of wall time (one second unless
// the knob says otherwise: a copy that has not landed after that long never will); false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint64_t limit_ns) {
  const uint32_t a = smem_addr(bar);
  uint64_t deadline = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(a), "r"(parity)
        : "memory");
    if (done) return true;
    if (i >= 64) {  // past the common latency: back off and watch the clock
      __nanosleep(64);
      const uint64_t now = global_timer_ns();
      if (deadline == 0)
        deadline = now + limit_ns;
      else if (now > deadline)
        return false;
    }
  }
}
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store(void *gdst, const void *smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

struct BulkParams {
  GatherPagesParams g;  // kSeg = false geometry; part_vecs * 16 <= stage_bytes
  int32_t stage_bytes, stages, pipes, lag;
  int64_t wait_ns;     // limit of every wait on a copy
  int32_t test_stall;  // test hook, see kvx_gather_bulk_kernel
};

template <typename IdxT>
__global__ void __launch_bounds__(kGatherThreads) kvx_gather_bulk_kernel(const BulkParams bp) {
  const GatherPagesParams &p = bp.g;
  extern __shared__ __align__(128) unsigned char s_raw[];
  __shared__ int32_t s_warp_tot[kGatherWarps];
  __shared__ __align__(8) uint64_t s_bar[kBulkMaxPipes * kBulkMaxStages + 1];
  // layout of dynamic shared memory: [stages of all pipes][prefix]
  unsigned char *stage_mem = s_raw;
  int32_t *s_prefix =
      reinterpret_cast<int32_t *>(s_raw + static_cast<size_t>(bp.pipes) * bp.stages * bp.stage_bytes);

  if (threadIdx.x <= kBulkMaxPipes * kBulkMaxStages) mbar_init(&s_bar[threadIdx.x], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  int64_t chunks;
  if (p.use_prefix)
    chunks = build_page_prefix<IdxT>(p, s_prefix, s_warp_tot);  // ends with __syncthreads()
  else {
    chunks = static_cast<int64_t>(p.s.seq_count) * p.s.max_blocks;
    __syncthreads();
  }

  const int warp_in_cta = threadIdx.x >> 5;
  if ((threadIdx.x & 31) != 0 || warp_in_cta >= bp.pipes) return;  // one elected thread per pipe

  const int64_t pipe = static_cast<int64_t>(blockIdx.x) * bp.pipes + warp_in_cta;
  const int64_t npipes = static_cast<int64_t>(gridDim.x) * bp.pipes;
  const int64_t items = chunks * p.parts * 2;
  unsigned char *my_stage = stage_mem + static_cast<size_t>(warp_in_cta) * bp.stages * bp.stage_bytes;
  uint64_t *my_bar = &s_bar[warp_in_cta * kBulkMaxStages];

  // Ring bookkeeping.  Item n of this pipe uses stage n % stages; its load completes phase
  // (n / stages) & 1 of that stage's barrier.  Loads run `lag` items ahead of stores, so a
  // pipe has `lag` loads and up to `stages - lag` stores in flight.
  char *dst_q[kBulkMaxStages] = {};
  uint32_t bytes_q[kBulkMaxStages] = {};
  int64_t issued = 0, retired = 0;
  bool failed = false;
  // Test hook for the give-up path: the first pipe of the grid waits on the spare barrier, for
  // which no copy was ever issued, before it has issued anything itself.  The wait runs out,
  // the pipe reports and leaves with nothing in flight; its work items stay undone.
  if (bp.test_stall && pipe == 0)
    failed = !mbar_wait(&s_bar[kBulkMaxPipes * kBulkMaxStages], 0, static_cast<uint64_t>(bp.wait_ns));

  auto retire_one = [&]() {
    const int st = static_cast<int>(retired % bp.stages);
    const uint32_t parity = static_cast<uint32_t>((retired / bp.stages) & 1);
    if (!mbar_wait(&my_bar[st], parity, static_cast<uint64_t>(bp.wait_ns))) {
      failed = true;
      return;
    }
    bulk_store(dst_q[st], my_stage + static_cast<size_t>(st) * bp.stage_bytes, bytes_q[st]);
    ++retired;
  };

  for (int64_t item = pipe; item < items && !failed; item += npipes) {
    const int kv = static_cast<int>(item & 1);
    const int64_t rest = item >> 1;
    const int64_t c = rest / p.parts;
    const int part = static_cast<int>(rest - c * p.parts);
    ChunkRef ref;
    if (p.use_prefix) {
      ref = find_chunk(s_prefix, p.s.seq_count, static_cast<int32_t>(c));
    } else {
      ref.seq = static_cast<int32_t>(c / p.s.max_blocks);
      ref.lb = static_cast<int32_t>(c - static_cast<int64_t>(ref.seq) * p.s.max_blocks);
    }
    const ChunkInfo ci = resolve_chunk<IdxT>(p, ref.seq, ref.lb);
    if (ci.block < 0) continue;
    const int64_t nbytes = static_cast<int64_t>(ci.tokens) * p.out_row_bytes;
    const int64_t bbeg = static_cast<int64_t>(part) * p.part_vecs * 16;
    if (bbeg >= nbytes) continue;
    const uint32_t bytes = static_cast<uint32_t>(min(static_cast<int64_t>(p.part_vecs) * 16, nbytes - bbeg));
    const char *src = (kv ? p.v_base + ci.block * p.v_blk : p.k_base + ci.block * p.k_blk) + bbeg;
    char *dst = (kv ? p.value_out : p.key_out) + ci.out_off + bbeg;

    // Keep at most `lag` loads outstanding: drain the oldest into a store first.
    if (issued - retired >= bp.lag) retire_one();
    if (failed) break;
    const int st = static_cast<int>(issued % bp.stages);
    // The stage was last read by the store of item `issued - stages`.  Stores are committed
    // in item order and `issued - lag + 1` of them exist now, so `stages - lag` groups were
    // committed after that one: once at most that many are still reading, it is done.
    switch (bp.stages - bp.lag) {
      case 0: bulk_wait_read<0>(); break;
      case 1: bulk_wait_read<1>(); break;
      case 2: bulk_wait_read<2>(); break;
      case 3: bulk_wait_read<3>(); break;
      case 4: bulk_wait_read<4>(); break;
      case 5: bulk_wait_read<5>(); break;
      case 6: bulk_wait_read<6>(); break;
      default: bulk_wait_read<7>(); break;
    }
    mbar_expect_tx(&my_bar[st], bytes);
    bulk_load(my_stage + static_cast<size_t>(st) * bp.stage_bytes, src, bytes, &my_bar[st]);
    dst_q[st] = dst;
    bytes_q[st] = bytes;
    ++issued;
  }
  while (retired < issued && !failed) retire_one();
  if (failed) atomicExch(&g_device_error, 1);
  bulk_wait_all();  // stores must complete before shared memory is released
}

// ------------------------------------------------------------------ absmax -> scale ----

constexpr int kScaleThreads = 256;

struct ScalesParams {
  const char *key, *value;
  int64_t total_vecs;  // 16-byte vectors per tensor
  int32_t vpr, vpr_shift, vps, vps_shift;
  int32_t heads;
  int32_t group;       // lanes that share one head in every iteration (power of two <= 32)
  int32_t per_tensor;  // 1: one scale per tensor
  float *k_out, *v_out;
  uint32_t *work;  // [2 * heads] running maxima (magnitude bits) + [1] CTA ticket
};

// |x| as f32 bits, maximum over the elements of one 16-byte vector.
__device__ __forceinline__ uint32_t absmax_vec(const uint4 &x, BF16) {
  const uint32_t a = __vmaxu2(__vmaxu2(x.x & 0x7FFF7FFFu, x.y & 0x7FFF7FFFu),
                              __vmaxu2(x.z & 0x7FFF7FFFu, x.w & 0x7FFF7FFFu));
  return max(a & 0xFFFFu, a >> 16) << 16;
}
__device__ __forceinline__ uint32_t absmax_vec(const uint4 &x, F16) {
  const uint32_t a = __vmaxu2(__vmaxu2(x.x & 0x7FFF7FFFu, x.y & 0x7FFF7FFFu),
                              __vmaxu2(x.z & 0x7FFF7FFFu, x.w & 0x7FFF7FFFu));
  const uint16_t m = static_cast<uint16_t>(max(a & 0xFFFFu, a >> 16));  // order-preserving on |f16|
  return __float_as_uint(__half2float(__ushort_as_half(m))) & 0x7FFFFFFFu;
}
__device__ __forceinline__ uint32_t absmax_vec(const uint4 &x, F32) {
  return max(max(x.x & 0x7FFFFFFFu, x.y & 0x7FFFFFFFu), max(x.z & 0x7FFFFFFFu, x.w & 0x7FFFFFFFu));
}

// kFixedHead (token rows of a power-of-two number of vectors): a thread keeps its place in the
// token row -- the same head -- in every iteration, so it keeps its maxima in registers, four
// loads of K and of V in flight, and joins the other lanes of its head once, after the loop
// (the kernel is otherwise bound by instruction issue, not by memory).
template <typename IoT, bool kFixedHead>
__global__ void __launch_bounds__(kScaleThreads) kvx_kv_scales_kernel(const ScalesParams p) {
  extern __shared__ uint32_t s_max[];  // [2 * heads]
  __shared__ int s_last;
  const int tid = threadIdx.x;
  for (int i = tid; i < 2 * p.heads; i += kScaleThreads) s_max[i] = 0;
  __syncthreads();

  const int64_t stride = static_cast<int64_t>(gridDim.x) * kScaleThreads;
  if constexpr (kFixedHead) {
    // A CTA owns a contiguous range of token rows and, of each row, either all of it (rows of up
    // to 256 vectors: 256 / vpr rows per iteration) or one block of 256 vectors (longer rows):
    // a thread keeps its place in the row, memory is walked front to back.
    const int col_blocks = p.vpr > kScaleThreads ? p.vpr / kScaleThreads : 1;
    const int rows_per_iter = p.vpr < kScaleThreads ? kScaleThreads / p.vpr : 1;
    const int col = static_cast<int>(blockIdx.x % col_blocks) * kScaleThreads + (p.vpr < kScaleThreads ? tid % p.vpr : tid);
    const int64_t chunks = gridDim.x / col_blocks;  // the launcher makes the grid a multiple of col_blocks
    const int64_t rows = p.total_vecs / p.vpr;
    const int64_t per_chunk = (rows + chunks - 1) / chunks;
    const int64_t chunk = blockIdx.x / col_blocks;
    const int64_t end = min(rows, (chunk + 1) * per_chunk);
    uint32_t mk = 0, mv = 0;
    int64_t r = chunk * per_chunk + (p.vpr < kScaleThreads ? tid / p.vpr : 0);
    const int64_t step = static_cast<int64_t>(rows_per_iter) * p.vpr;  // vectors between a thread's iterations
    int64_t f = r * p.vpr + col;
    for (; r + 3 * rows_per_iter < end; r += 4 * rows_per_iter, f += 4 * step) {
      uint4 a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a[u] = load_stream(p.key + (f + u * step) * 16);
        b[u] = load_stream(p.value + (f + u * step) * 16);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        mk = max(mk, absmax_vec(a[u], IoT{}));
        mv = max(mv, absmax_vec(b[u], IoT{}));
      }
    }
    for (; r < end; r += rows_per_iter, f += step) {
      mk = max(mk, absmax_vec(load_stream(p.key + f * 16), IoT{}));
      mv = max(mv, absmax_vec(load_stream(p.value + f * 16), IoT{}));
    }
    // lanes of one group share a head (the group divides the vectors per head and a warp's
    // columns are consecutive and aligned): fold them, then one shared-memory update each
    for (int d = 1; d < p.group; d <<= 1) {
      mk = max(mk, __shfl_xor_sync(0xFFFFFFFFu, mk, d));
      mv = max(mv, __shfl_xor_sync(0xFFFFFFFFu, mv, d));
    }
    if ((tid & (p.group - 1)) == 0) {
      const int h = div_by(col, p.vps, p.vps_shift);
      if (mk) atomicMax(&s_max[h], mk);
      if (mv) atomicMax(&s_max[p.heads + h], mv);
    }
  } else {
    // total_vecs is rounded up to a multiple of the CTA size by the loop bound so that every
    // lane of a warp takes part in the shuffles.
    const int64_t bound = (p.total_vecs + kScaleThreads - 1) / kScaleThreads * kScaleThreads;
    for (int64_t f = static_cast<int64_t>(blockIdx.x) * kScaleThreads + tid; f < bound; f += stride) {
      uint32_t mk = 0, mv = 0;
      int h = 0;
      if (f < p.total_vecs) {
        mk = absmax_vec(load_stream(p.key + f * 16), IoT{});
        mv = absmax_vec(load_stream(p.value + f * 16), IoT{});
        const int v = static_cast<int>(p.vpr_shift >= 0 ? (f & (p.vpr - 1)) : (f % p.vpr));
        h = div_by(v, p.vps, p.vps_shift);
      }
      for (int d = 1; d < p.group; d <<= 1) {
        mk = max(mk, __shfl_xor_sync(0xFFFFFFFFu, mk, d));
        mv = max(mv, __shfl_xor_sync(0xFFFFFFFFu, mv, d));
      }
      if ((tid & (p.group - 1)) == 0 && f < p.total_vecs) {
        if (mk) atomicMax(&s_max[h], mk);
        if (mv) atomicMax(&s_max[p.heads + h], mv);
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < 2 * p.heads; i += kScaleThreads)
    if (s_max[i]) atomicMax(&p.work[i], s_max[i]);
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = (atomicAdd(&p.work[2 * p.heads], 1u) == gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Last CTA: turn the maxima into scales and leave the workspace zeroed for the next call.
  if (p.per_tensor) {
    if (tid < 2) {
      uint32_t m = 0;
      for (int hh = 0; hh < p.heads; ++hh) m = max(m, __ldcg(&p.work[tid * p.heads + hh]));
      const float s = __fdiv_rn(__uint_as_float(m), 448.0f);
      (tid == 0 ? p.k_out : p.v_out)[0] = (s > 0.0f) ? s : 1.0f;
    }
  } else {
    for (int i = tid; i < 2 * p.heads; i += kScaleThreads) {
      const float s = __fdiv_rn(__uint_as_float(__ldcg(&p.work[i])), 448.0f);
      (i < p.heads ? p.k_out : p.v_out)[i < p.heads ? i : i - p.heads] = (s > 0.0f) ? s : 1.0f;
    }
  }
  __syncthreads();
  for (int i = tid; i <= 2 * p.heads; i += kScaleThreads) p.work[i] = 0;
}

// ------------------------------------------------------------------ host: validation ---

// IO tensor shape / stride checks of the launchers (reference: kernels/kvx_paged_kv.cu:269-313).
kvx_status_t check_io_tensor(const kvx_tensor_desc_t *t, uint32_t ndim, const int64_t *dims) {
  if (t->ndim != ndim) return KVX_STATUS_INVALID_ARGUMENT;
  for (uint32_t i = 0; i < ndim; ++i)
    if (t->shape[i] != dims[i]) return KVX_STATUS_INVALID_ARGUMENT;
  int64_t run = 1;
  for (uint32_t i = ndim; i-- > 0;) {
    if (t->stride[i] != run) return KVX_STATUS_UNSUPPORTED;
    run *= dims[i];
  }
  return KVX_STATUS_OK;
}

// The write's key / value: as check_io_tensor, except that token rows may lie further apart
// than heads * dim elements (a slice of a fused projection output, which is what vLLM hands its
// own cache-write operator).  The reference asks for dense rows (kernels/kvx_paged_kv.cu:269-313)
// and answers UNSUPPORTED; everything else about the tensor is checked as it does.
kvx_status_t check_write_rows(const kvx_tensor_desc_t *t, const int64_t *dims) {
  if (t->ndim != 3) return KVX_STATUS_INVALID_ARGUMENT;
  for (uint32_t i = 0; i < 3; ++i)
    if (t->shape[i] != dims[i]) return KVX_STATUS_INVALID_ARGUMENT;
  if (t->stride[2] != 1 || t->stride[1] != dims[2] || t->stride[0] < dims[1] * dims[2]) return KVX_STATUS_UNSUPPORTED;
  return KVX_STATUS_OK;
}

bool io_dtype_quantisable(kvx_dtype_t t) {
  return t == KVX_DTYPE_F16 || t == KVX_DTYPE_BF16 || t == KVX_DTYPE_F32;
}

cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

kvx_status_t finish_launch() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? KVX_STATUS_OK : KVX_STATUS_INTERNAL_ERROR;
}

// Launch with (or without) the programmatic-stream-serialization attribute.
template <typename Params>
void launch_streaming(void (*kernel)(Params), unsigned grid, unsigned block, size_t smem, cudaStream_t st,
                      const Params &p) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = opt(g_opt.pdl) ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, p);
}

// ------------------------------------------------------------------ host: write --------

template <typename SlotT, bool kSeg>
void launch_write_rows(const WriteRowsParams &p, int grid, int unroll, cudaStream_t st) {
  if (unroll >= 4)
    launch_streaming(kvx_write_rows_kernel<SlotT, kSeg, 4>, grid, kWriteThreads, 0, st, p);
  else if (unroll >= 2)
    launch_streaming(kvx_write_rows_kernel<SlotT, kSeg, 2>, grid, kWriteThreads, 0, st, p);
  else
    launch_streaming(kvx_write_rows_kernel<SlotT, kSeg, 1>, grid, kWriteThreads, 0, st, p);
}

template <typename IoT, typename CacheT>
kvx_status_t launch_write_generic(const kvx_write_desc_t *w, const GenericParams &gp, cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(w->io.num_tokens) * gp.g.heads * gp.g.dim;
  const int64_t grid = (total + 255) / 256;
  if (grid > INT32_MAX) return KVX_STATUS_UNSUPPORTED;
  const IoT *k = static_cast<const IoT *>(w->io.key.data);
  const IoT *v = static_cast<const IoT *>(w->io.value.data);
  if (w->slots.dtype == KVX_DTYPE_S32)
    kvx_write_generic_kernel<IoT, CacheT, int32_t>
        <<<static_cast<unsigned>(grid), 256, 0, st>>>(k, v, w->io.key.stride[0], w->io.value.stride[0], w->slots.slots,
                                                      w->io.num_tokens, gp);
  else
    kvx_write_generic_kernel<IoT, CacheT, int64_t>
        <<<static_cast<unsigned>(grid), 256, 0, st>>>(k, v, w->io.key.stride[0], w->io.value.stride[0], w->slots.slots,
                                                      w->io.num_tokens, gp);
  return finish_launch();
}

// Tokens per CTA: aim at `write_vecs_per_cta` vectors of K per CTA, but never fewer CTAs
// than fill the machine twice when the batch is small.
// CTAs of a warp-item gather kernel.  Work items are small (one unrolled iteration of a warp)
// and there are many more CTAs than fit at once, so the hardware scheduler balances the tail;
// measured best at up to `per_sm` = 256 CTAs per SM, but never more than half a CTA-slot per item
// of the padded (sequence, page) rectangle: beyond that most CTAs would only run their prefix
// scan.  A rectangle of more than 65 536 (sequence, page) pairs is a batch of contexts padded to
// the longest one, mostly holes (a decode batch of 512 contexts of 1 to 1 024 pages is 9 % full):
// it is counted as 65 536 pairs and given four items per warp, not two, because every CTA pays
// the scan over all sequences before its first item (one head of 8, full contexts of that
// batch: 285 us with 256 CTAs per SM, 233 us with 64).
int64_t gather_item_grid(int64_t seq_count, int64_t max_blocks, int64_t items_per_chunk, int sm_count, int64_t per_sm,
                         int warps_per_cta) {
  const int64_t rect = seq_count * max_blocks;
  const bool sparse = rect > 65536;
  const int64_t items = (sparse ? int64_t{65536} : rect) * items_per_chunk;
  const int64_t ctas = (items + warps_per_cta - 1) / warps_per_cta;
  return std::max<int64_t>(1, std::min(static_cast<int64_t>(sm_count) * per_sm, (ctas + 1) / (sparse ? 4 : 2)));
}

int pick_tok_tile(int64_t tokens, int64_t vpr, int sm_count) {
  int64_t tile = opt(g_opt.write_vecs_per_cta) / vpr;
  if (tile < 1) tile = 1;
  if (tile > kMaxTokTile) tile = kMaxTokTile;
  const int64_t want_ctas = static_cast<int64_t>(sm_count) * 4;
  while (tile > 1 && (tokens + tile - 1) / tile < want_ctas) tile >>= 1;
  return static_cast<int>(tile);
}

/*
 * Shared body of every write entry point.  `expected` is the cache dtype the entry point
 * is pinned to; for F8_E4M3 the IO tensors may be F16 / BF16 / F32.
 * Check order: reference kernels/kvx_paged_kv.cu:320-376 (write), :497-559 (prefill).
 */
kvx_status_t write_impl(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write, void *stream,
                        kvx_dtype_t expected, bool prefill, int32_t tokens_per_seq) {
  if (cache == nullptr || write == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (prefill && tokens_per_seq <= 0) return KVX_STATUS_INVALID_ARGUMENT;
  if (write->size < sizeof(kvx_write_desc_t) || write->io.size < sizeof(kvx_kv_io_desc_t) ||
      write->slots.size < sizeof(kvx_slot_mapping_t))
    return KVX_STATUS_INVALID_ARGUMENT;
  if (prefill && (write->io.num_tokens % static_cast<uint32_t>(tokens_per_seq)) != 0)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype != expected || cache->v.dtype != expected) return KVX_STATUS_UNSUPPORTED;
  const bool fp8 = (expected == KVX_DTYPE_F8_E4M3);
  const kvx_dtype_t io_dtype = write->io.key.dtype;
  ScaleView ks{nullptr, 0}, vs{nullptr, 0};
  if (fp8) {
    if (!io_dtype_quantisable(io_dtype) || write->io.value.dtype != io_dtype) return KVX_STATUS_UNSUPPORTED;
    if (!resolve_scale(&write->k_scale_desc, write->k_scale, cache->num_kv_heads, &ks) ||
        !resolve_scale(&write->v_scale_desc, write->v_scale, cache->num_kv_heads, &vs))
      return KVX_STATUS_UNSUPPORTED;
  } else if (io_dtype != expected || write->io.value.dtype != expected) {
    return KVX_STATUS_UNSUPPORTED;
  }
  if (write->io.num_kv_heads != cache->num_kv_heads || write->io.head_dim != cache->head_dim)
    return KVX_STATUS_INVALID_ARGUMENT;
  const int64_t dims[3] = {write->io.num_tokens, write->io.num_kv_heads, write->io.head_dim};
  kvx_status_t st = check_write_rows(&write->io.key, dims);
  if (st != KVX_STATUS_OK) return st;
  st = check_write_rows(&write->io.value, dims);
  if (st != KVX_STATUS_OK) return st;
  if (write->slots.token_count != write->io.num_tokens) return KVX_STATUS_INVALID_ARGUMENT;

  const int64_t elem = dtype_bytes(expected);
  const int64_t io_elem = dtype_bytes(io_dtype);
  GenericParams gp;
  st = make_page_view(cache, &cache->k, elem, &gp.k);
  if (st != KVX_STATUS_OK) return st;
  st = make_page_view(cache, &cache->v, elem, &gp.v);
  if (st != KVX_STATUS_OK) return st;
  gp.g = Geometry{static_cast<int32_t>(cache->num_blocks), static_cast<int32_t>(cache->block_size),
                  static_cast<int32_t>(cache->num_kv_heads), static_cast<int32_t>(cache->head_dim),
                  static_cast<int32_t>(elem)};
  gp.ks = ks;
  gp.vs = vs;

  const int64_t T = write->io.num_tokens, H = cache->num_kv_heads, D = cache->head_dim;
  if (T * H * D == 0) return KVX_STATUS_OK;
  if (write->slots.dtype != KVX_DTYPE_S32 && write->slots.dtype != KVX_DTYPE_S64)
    return KVX_STATUS_INVALID_ARGUMENT;
  // Stricter than the reference, which would fault on the device instead.
  if (write->io.key.data == nullptr || write->io.value.data == nullptr || write->slots.slots == nullptr ||
      cache->k.data == nullptr || cache->v.data == nullptr || cache->block_size == 0 ||
      cache->num_blocks > static_cast<uint32_t>(INT32_MAX) || T > INT32_MAX)
    return KVX_STATUS_INVALID_ARGUMENT;

  const cudaStream_t cs = as_stream(stream);
  const DeviceInfo &dev = device_info();
  const bool s32 = (write->slots.dtype == KVX_DTYPE_S32);

  // ---- vector tier: 16-byte input vectors, each inside one head -------------------------
  const int64_t row_bytes = H * D * io_elem;
  const int64_t out_vec = fp8 ? 16 / io_elem : 16;  // cache bytes produced per input vector
  int32_t k_sub = 0, v_sub = 0;
  const bool k_packed = !fp8 && view_packed16(gp.k, elem, D, &k_sub), v_packed = !fp8 && view_packed16(gp.v, elem, D, &v_sub);
  const int64_t k_pitch = write->io.key.stride[0] * io_elem, v_pitch = write->io.value.stride[0] * io_elem;
  const bool pitched = k_pitch != row_bytes || v_pitch != row_bytes;  // token rows further apart than dense
  // ---- packed pages with pack groups below 16 bytes (or mixed): fragment / transposition tier --
  PackedSide k_side{}, v_side{};
  const int64_t tiles_knob = opt(g_opt.packed_tiles);
  if (!fp8 && !opt(g_opt.force_generic) && tiles_knob != 0 && (D * io_elem) % 16 == 0 && k_pitch % 16 == 0 &&
      v_pitch % 16 == 0 && aligned(write->io.key.data, 16) && aligned(write->io.value.data, 16) &&
      row_bytes / 16 <= (1 << 20) && view_packed_tile(gp.k, elem, D, cache->block_size, &k_side) &&
      view_packed_tile(gp.v, elem, D, cache->block_size, &v_side) &&
      // K and V both in 16-byte groups: whole-line fragments when the shape allows (a multiple of 8
      // groups per head, pages of a multiple of 8 tokens), else the token-fastest row kernel below
      (k_side.n_shift != 0 || v_side.n_shift != 0 || tiles_knob == 2 ||
       (tiles_knob != 3 && (D * io_elem) % 128 == 0 && cache->block_size % 8 == 0))) {
    WritePackedParams q;
    q.key = static_cast<const char *>(write->io.key.data);
    q.value = static_cast<const char *>(write->io.value.data);
    q.k_pitch = k_pitch, q.v_pitch = v_pitch;
    q.k_base = gp.k.base, q.k_blk = gp.k.blk, q.k_head = gp.k.head;
    q.v_base = gp.v.base, q.v_blk = gp.v.blk, q.v_head = gp.v.head;
    q.k = k_side, q.v = v_side;
    q.slots = write->slots.slots;
    q.num_tokens = static_cast<int32_t>(T);
    q.num_blocks = gp.g.num_blocks;
    q.block_size = gp.g.block_size;
    q.bs_shift = shift_of(q.block_size);
    q.vpr = static_cast<int32_t>(row_bytes / 16);
    q.vph = static_cast<int32_t>(D * io_elem / 16);
    q.vph_shift = shift_of(q.vph);
    // Tokens per CTA: the knob's value for token rows of 2 KB (8 heads x 128 x 16 bits) and more,
    // proportionally more tokens for shorter rows (a shard of the heads), so that a CTA's set-up
    // (slots, fragment lists) is spread over about as many bytes.
    int64_t want = std::max<int64_t>(1, opt(g_opt.packed_tile_tokens));
    if (row_bytes < 2048) want = want * 2048 / std::max<int64_t>(row_bytes, 16);
    int tile = static_cast<int>(std::min<int64_t>(kPackedTile, want));
    while ((tile & (tile - 1)) != 0) tile &= tile - 1;  // a power of two
    while (tile > 1 && (T + tile - 1) / tile < static_cast<int64_t>(dev.sm_count) * 4) tile >>= 1;
    q.tok_tile = tile;
    const bool lines_shape = tiles_knob != 2 && tiles_knob != 3 && (D * io_elem) % 128 == 0 && cache->block_size % 8 == 0;
    // (K alone through the whole-line routine next to a V of 2-byte units measured slower than K
    // as two-slot fragments: 5.28 against 5.61 TB/s on the paged Llama-3-70B shape)
    q.k_lines = q.v_lines = lines_shape && k_side.n_shift == 0 && v_side.n_shift == 0;
    q.fill_halves = opt(g_opt.packed_fill_halves) != 0;
    const int grid = static_cast<int>((T + tile - 1) / tile);
    if (q.k_lines && q.v_lines) {
      const int64_t variant = opt(g_opt.packed_lines_variant);
#define KVX_LINES(ROUND, CTAS)                                                                                  \
  do {                                                                                                          \
    if (s32)                                                                                                    \
      launch_streaming(kvx_write_packed_lines_kernel<int32_t, ROUND, CTAS>, grid, kWriteThreads, 0, cs, q);     \
    else                                                                                                        \
      launch_streaming(kvx_write_packed_lines_kernel<int64_t, ROUND, CTAS>, grid, kWriteThreads, 0, cs, q);     \
  } while (0)
      // Two rounds of loads per thread at 40 registers and 6 CTAs per SM, or four at 64 and 4:
      // measured equal within 2 % on full batches (5.92-5.97 against 5.81-5.96 TB/s unpadded, 4.04
      // against 4.08 TB/s with 10 % padded slots), the first 5 % ahead on a one-head shard.  With
      // spills to reach 5 or 8 CTAs per SM it is 10-20 % slower.
      if (variant == 1)
        KVX_LINES(4, 4);
      else
        KVX_LINES(2, 6);
#undef KVX_LINES
      return finish_launch();
    }
    if (s32)
      launch_streaming(kvx_write_packed_kernel<int32_t>, grid, kWriteThreads, 0, cs, q);
    else
      launch_streaming(kvx_write_packed_kernel<int64_t>, grid, kWriteThreads, 0, cs, q);
    return finish_launch();
  }
  const bool vec_ok = !opt(g_opt.force_generic) && (D * io_elem) % 16 == 0 && k_pitch % 16 == 0 && v_pitch % 16 == 0 &&
                      !(pitched && (k_packed || v_packed)) &&
                      (!fp8 || (gp.k.head * H < INT32_MAX && gp.v.head * H < INT32_MAX)) &&  // 32-bit in-page offsets
                      aligned(write->io.key.data, 16) && aligned(write->io.value.data, 16) &&
                      (k_packed || view_vectorisable(gp.k, elem, D, out_vec)) &&
                      (v_packed || view_vectorisable(gp.v, elem, D, out_vec)) && row_bytes / 16 <= (1 << 20);
  if (vec_ok) {
    WriteRowsParams p;
    p.key = static_cast<const char *>(write->io.key.data);
    p.value = static_cast<const char *>(write->io.value.data);
    p.k_base = gp.k.base, p.k_blk = gp.k.blk, p.k_tok = gp.k.tok, p.k_head = gp.k.head;
    p.v_base = gp.v.base, p.v_blk = gp.v.blk, p.v_tok = gp.v.tok, p.v_head = gp.v.head;
    p.k_vec = k_packed ? gp.k.dhi : 16, p.v_vec = v_packed ? gp.v.dhi : 16;
    p.k_sub = k_sub, p.v_sub = v_sub;
    p.slots = write->slots.slots;
    p.row_bytes = row_bytes;
    p.k_pitch = k_pitch, p.v_pitch = v_pitch;
    p.num_tokens = static_cast<int32_t>(T);
    p.num_blocks = gp.g.num_blocks;
    p.block_size = gp.g.block_size;
    p.bs_shift = shift_of(p.block_size);
    p.vpr = static_cast<int32_t>(row_bytes / 16);
    p.vpr_shift = shift_of(p.vpr);
    p.vps = static_cast<int32_t>(D * io_elem / 16);
    p.vps_shift = shift_of(p.vps);
    p.tok_tile = pick_tok_tile(T, p.vpr, dev.sm_count);
    p.tile_shift = 0;
    if (k_packed || v_packed) {
      // Token-fastest order over tiles of 16 tokens: a warp then covers 16 consecutive slots x
      // 2 pack groups, i.e. two 256-byte runs of a page on the store side and whole 32-byte
      // sectors of 16 token rows on the load side (measured: 6 231 GB/s on the unpadded
      // Llama-3-70B shape; with 10 % of the slots padded the holes in the runs make the
      // memory system merge partial sectors and the rate drops to 2.9 TB/s).
      int tile = 16;
      while (tile > 1 && (T + tile - 1) / tile < static_cast<int64_t>(dev.sm_count) * 4) tile >>= 1;
      p.tok_tile = tile;
      p.tile_shift = shift_of(tile);
    }
    const int grid = static_cast<int>((T + p.tok_tile - 1) / p.tok_tile);
    const int unroll = static_cast<int>(opt(g_opt.write_unroll));
    // Leading CTAs that prefetch (see write_prologue): worth 1 us on a launch of a few tens of
    // microseconds, nothing on a long one, where back-to-back writes even lose 1 % to the early
    // requests competing with the previous launch's last stores -- so only grids of up to twice
    // that many CTAs use it.
    const int64_t lead = static_cast<int64_t>(dev.sm_count) * 8 * opt(g_opt.write_prefetch_waves);
    p.early_ctas = grid <= 2 * lead ? static_cast<int32_t>(std::min<int64_t>(lead, INT32_MAX)) : 0;
    if (fp8) {
      WriteF8Params q{p, ks, vs, static_cast<int32_t>(D), static_cast<int32_t>(H)};
      // 256-bit variant: 16-bit inputs whose head rows are whole 32-byte vectors, dense and 32-byte
      // aligned, destinations 16-byte aligned, shapes powers of two
      const int64_t row32 = row_bytes / 32, head32 = D * io_elem / 32;
      if (opt(g_opt.wide) && io_elem == 2 && !pitched && (D * io_elem) % 32 == 0 && H <= kF8CachedHeads &&
          is_pow2(row32) && is_pow2(head32) && aligned(write->io.key.data, 32) && aligned(write->io.value.data, 32) &&
          aligned(gp.k.base, 16) && aligned(gp.v.base, 16) && gp.k.blk % 16 == 0 && gp.v.blk % 16 == 0 &&
          gp.k.tok % 16 == 0 && gp.v.tok % 16 == 0 && gp.k.head % 16 == 0 && gp.v.head % 16 == 0) {
        q.w.vpr = static_cast<int32_t>(row32), q.w.vpr_shift = shift_of(row32);
        q.w.vps = static_cast<int32_t>(head32), q.w.vps_shift = shift_of(head32);
        // 32-byte vectors per CTA: f8_tile_mult x the bytes per CTA of the 128-bit form
        const int64_t want = std::max<int64_t>(1, opt(g_opt.f8_tile_mult)) * opt(g_opt.write_vecs_per_cta) / 2;
        int64_t tile = std::min<int64_t>(kMaxTokTile, std::max<int64_t>(1, want / q.w.vpr));
        while (tile > 1 && (T + tile - 1) / tile < static_cast<int64_t>(dev.sm_count) * 4) tile >>= 1;
        q.w.tok_tile = static_cast<int32_t>(tile);
        const int wgrid = static_cast<int>((T + q.w.tok_tile - 1) / q.w.tok_tile);
        const bool two = opt(g_opt.f8_unroll) >= 2;
#define KVX_F8_WIDE(IoT, SlotT)                                                                   \
  do {                                                                                            \
    if (two)                                                                                      \
      launch_streaming(kvx_write_f8_wide_kernel<IoT, SlotT, 2>, wgrid, kWriteThreads, 0, cs, q);  \
    else                                                                                          \
      launch_streaming(kvx_write_f8_wide_kernel<IoT, SlotT, 1>, wgrid, kWriteThreads, 0, cs, q);  \
  } while (0)
        if (io_dtype == KVX_DTYPE_BF16) {
          if (s32)
            KVX_F8_WIDE(BF16, int32_t);
          else
            KVX_F8_WIDE(BF16, int64_t);
        } else {
          if (s32)
            KVX_F8_WIDE(F16, int32_t);
          else
            KVX_F8_WIDE(F16, int64_t);
        }
#undef KVX_F8_WIDE
        return finish_launch();
      }
#define KVX_F8_WRITE(IoT)                                                                                     \
  do {                                                                                                        \
    if (pitched) {                                                                                            \
      if (s32)                                                                                                \
        launch_streaming(kvx_write_f8_kernel<IoT, int32_t, KVX_F8_WRITE_UNROLL, true>, grid, kWriteThreads, 0, cs, q); \
      else                                                                                                    \
        launch_streaming(kvx_write_f8_kernel<IoT, int64_t, KVX_F8_WRITE_UNROLL, true>, grid, kWriteThreads, 0, cs, q); \
    } else if (p.vpr_shift >= 0 && p.vps_shift >= 0) {                                                        \
      if (s32)                                                                                                \
        launch_streaming(kvx_write_f8_kernel<IoT, int32_t, KVX_F8_WRITE_UNROLL, false, true>, grid, kWriteThreads, 0, cs, q); \
      else                                                                                                    \
        launch_streaming(kvx_write_f8_kernel<IoT, int64_t, KVX_F8_WRITE_UNROLL, false, true>, grid, kWriteThreads, 0, cs, q); \
    } else if (s32) {                                                                                         \
      launch_streaming(kvx_write_f8_kernel<IoT, int32_t, KVX_F8_WRITE_UNROLL>, grid, kWriteThreads, 0, cs, q); \
    } else {                                                                                                  \
      launch_streaming(kvx_write_f8_kernel<IoT, int64_t, KVX_F8_WRITE_UNROLL>, grid, kWriteThreads, 0, cs, q); \
    }                                                                                                         \
  } while (0)
      if (io_dtype == KVX_DTYPE_BF16)
        KVX_F8_WRITE(BF16);
      else if (io_dtype == KVX_DTYPE_F16)
        KVX_F8_WRITE(F16);
      else
        KVX_F8_WRITE(F32);
#undef KVX_F8_WRITE
      return finish_launch();
    }
    const bool seg = k_packed || v_packed || !(gp.k.head == D * elem && gp.v.head == D * elem);
    if (k_packed || v_packed) {
      if (s32)
        launch_streaming(kvx_write_rows_kernel<int32_t, true, 4, true>, grid, kWriteThreads, 0, cs, p);
      else
        launch_streaming(kvx_write_rows_kernel<int64_t, true, 4, true>, grid, kWriteThreads, 0, cs, p);
      return finish_launch();
    }
    if (pitched) {
      if (s32)
        launch_streaming(kvx_write_rows_kernel<int32_t, true, 4, false, true>, grid, kWriteThreads, 0, cs, p);
      else
        launch_streaming(kvx_write_rows_kernel<int64_t, true, 4, false, true>, grid, kWriteThreads, 0, cs, p);
      return finish_launch();
    }
    if (s32) {
      if (seg)
        launch_write_rows<int32_t, true>(p, grid, unroll, cs);
      else
        launch_write_rows<int32_t, false>(p, grid, unroll, cs);
    } else {
      if (seg)
        launch_write_rows<int64_t, true>(p, grid, unroll, cs);
      else
        launch_write_rows<int64_t, false>(p, grid, unroll, cs);
    }
    return finish_launch();
  }

  // ---- generic tier ---------------------------------------------------------------------
  if (fp8) {
    if (io_dtype == KVX_DTYPE_BF16) return launch_write_generic<BF16, F8>(write, gp, cs);
    if (io_dtype == KVX_DTYPE_F16) return launch_write_generic<F16, F8>(write, gp, cs);
    return launch_write_generic<F32, F8>(write, gp, cs);
  }
  if (elem == 2) return launch_write_generic<BF16, BF16>(write, gp, cs);  // 16-bit copy, either type
  return launch_write_generic<F32, F32>(write, gp, cs);
}

// ------------------------------------------------------------------ host: gather -------

template <typename IoT, typename CacheT, bool kDequant>
kvx_status_t launch_gather_generic(const kvx_gather_desc_t *g, const GatherShape &s, const GenericParams &gp,
                                   cudaStream_t st) {
  const int64_t total = static_cast<int64_t>(s.seq_count) * s.max_seq_len * gp.g.heads * gp.g.dim;
  const int64_t grid = (total + 255) / 256;
  if (grid > INT32_MAX) return KVX_STATUS_UNSUPPORTED;
  IoT *k = static_cast<IoT *>(g->io.key.data);
  IoT *v = static_cast<IoT *>(g->io.value.data);
  if (g->seq_lens.dtype == KVX_DTYPE_S32)
    kvx_gather_generic_kernel<IoT, CacheT, int32_t, kDequant>
        <<<static_cast<unsigned>(grid), 256, 0, st>>>(k, v, s, gp);
  else
    kvx_gather_generic_kernel<IoT, CacheT, int64_t, kDequant>
        <<<static_cast<unsigned>(grid), 256, 0, st>>>(k, v, s, gp);
  return finish_launch();
}

// Largest sequence count whose page-count prefix fits in shared memory next to everything
// else; beyond it the kernels walk the padded (sequence, page) rectangle instead.
constexpr int kMaxPrefixSeqs = 10240;

/*
 * Shared body of every gather entry point.
 * Check order: reference kernels/kvx_paged_kv.cu:768-829, :837-863.
 */
struct VarlenOut {  // un-padded output of kvx_launch_gather_kv_varlen
  const void *indptr;
  kvx_dtype_t dtype;
};

kvx_status_t gather_impl(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                         const kvx_scale_desc_t *k_scale, const kvx_scale_desc_t *v_scale, void *stream,
                         kvx_dtype_t expected, const VarlenOut *varlen = nullptr) {
  if (cache == nullptr || gather == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (gather->size < sizeof(kvx_gather_desc_t) || gather->io.size < sizeof(kvx_kv_io_desc_t) ||
      gather->block_table.size < sizeof(kvx_block_table_t) || gather->seq_lens.size < sizeof(kvx_seq_lens_t))
    return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype != expected || cache->v.dtype != expected) return KVX_STATUS_UNSUPPORTED;
  const bool fp8 = (expected == KVX_DTYPE_F8_E4M3);
  const kvx_dtype_t io_dtype = gather->io.key.dtype;
  ScaleView ks{nullptr, 0}, vs{nullptr, 0};
  if (fp8) {
    if (!io_dtype_quantisable(io_dtype) || gather->io.value.dtype != io_dtype) return KVX_STATUS_UNSUPPORTED;
    if (!resolve_scale(k_scale, nullptr, cache->num_kv_heads, &ks) ||
        !resolve_scale(v_scale, nullptr, cache->num_kv_heads, &vs))
      return KVX_STATUS_UNSUPPORTED;
  } else if (io_dtype != expected || gather->io.value.dtype != expected) {
    return KVX_STATUS_UNSUPPORTED;
  }
  // PACKED as in the reference; RAGGED (one page id per cached token, KVX_SPEC.md:108-114) is
  // executed here, the reference answers UNSUPPORTED for it (kernels/kvx_paged_kv.cu:788-790).
  // KV_OFFSETS (KVX_SPEC.md:116-122), also UNSUPPORTED in the reference, is executed for
  // beam_width 1: the output has one row per sequence, so there is no place for more beams.
  const bool ragged = gather->block_table.format == KVX_BLOCK_TABLE_RAGGED;
  const bool offsets = gather->block_table.format == KVX_BLOCK_TABLE_KV_OFFSETS;
  if (gather->block_table.format != KVX_BLOCK_TABLE_PACKED && !ragged && !offsets) return KVX_STATUS_UNSUPPORTED;
  if (gather->io.num_kv_heads != cache->num_kv_heads || gather->io.head_dim != cache->head_dim)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (gather->seq_lens.seq_count != gather->block_table.seq_count) return KVX_STATUS_INVALID_ARGUMENT;
  const int64_t dims[4] = {gather->block_table.seq_count, gather->max_seq_len, gather->io.num_kv_heads,
                           gather->io.head_dim};
  const int64_t flat[3] = {gather->io.num_tokens, gather->io.num_kv_heads, gather->io.head_dim};
  kvx_status_t st = varlen ? check_io_tensor(&gather->io.key, 3, flat) : check_io_tensor(&gather->io.key, 4, dims);
  if (st != KVX_STATUS_OK) return st;
  st = varlen ? check_io_tensor(&gather->io.value, 3, flat) : check_io_tensor(&gather->io.value, 4, dims);
  if (st != KVX_STATUS_OK) return st;
  if (varlen && (varlen->indptr == nullptr || (varlen->dtype != KVX_DTYPE_S32 && varlen->dtype != KVX_DTYPE_S64)))
    return KVX_STATUS_INVALID_ARGUMENT;

  const int64_t elem = dtype_bytes(expected);
  const int64_t io_elem = dtype_bytes(io_dtype);
  GenericParams gp;
  st = make_page_view(cache, &cache->k, elem, &gp.k);
  if (st != KVX_STATUS_OK) return st;
  st = make_page_view(cache, &cache->v, elem, &gp.v);
  if (st != KVX_STATUS_OK) return st;
  gp.g = Geometry{static_cast<int32_t>(cache->num_blocks), static_cast<int32_t>(cache->block_size),
                  static_cast<int32_t>(cache->num_kv_heads), static_cast<int32_t>(cache->head_dim),
                  static_cast<int32_t>(elem)};
  gp.ks = ks;
  gp.vs = vs;

  const int64_t S = gather->block_table.seq_count, L = gather->max_seq_len;
  const int64_t H = cache->num_kv_heads, D = cache->head_dim;
  if (S * L * H * D == 0 || (varlen && gather->io.num_tokens == 0)) return KVX_STATUS_OK;
  const bool s32 = gather->block_table.index_dtype == KVX_DTYPE_S32 && gather->seq_lens.dtype == KVX_DTYPE_S32;
  const bool s64 = gather->block_table.index_dtype == KVX_DTYPE_S64 && gather->seq_lens.dtype == KVX_DTYPE_S64;
  if (!s32 && !s64) return KVX_STATUS_INVALID_ARGUMENT;
  // Stricter than the reference, which would fault on the device instead.
  if (gather->io.key.data == nullptr || gather->io.value.data == nullptr ||
      gather->block_table.indices == nullptr || gather->seq_lens.lengths == nullptr ||
      cache->k.data == nullptr || cache->v.data == nullptr || cache->block_size == 0 ||
      gather->block_table.max_blocks_per_seq == 0 || cache->num_blocks > static_cast<uint32_t>(INT32_MAX) ||
      S > INT32_MAX || L > INT32_MAX || gather->block_table.max_blocks_per_seq > static_cast<uint32_t>(INT32_MAX))
    return KVX_STATUS_INVALID_ARGUMENT;

  GatherShape gs;
  gs.table = gather->block_table.indices;
  gs.lens = gather->seq_lens.lengths;
  gs.table_bytes = ragged ? 0
                          : static_cast<int64_t>(S) * gather->block_table.max_blocks_per_seq *
                                (offsets ? 8 : (gather->block_table.index_dtype == KVX_DTYPE_S64 ? 8 : 4));
  gs.seq_count = static_cast<int32_t>(S);
  gs.max_blocks = static_cast<int32_t>(gather->block_table.max_blocks_per_seq);
  gs.max_seq_len = static_cast<int32_t>(L);
  gs.indptr = nullptr;
  gs.indptr64 = 0;
  gs.indices_count = gather->block_table.indices_count;
  gs.pool[0] = gs.pool[1] = nullptr;
  gs.pool_block_bytes = 0;
  gs.beam_width = 1;
  gs.out_indptr = varlen ? varlen->indptr : nullptr;
  gs.out_indptr64 = varlen && varlen->dtype == KVX_DTYPE_S64;
  gs.out_rows = varlen ? static_cast<int64_t>(gather->io.num_tokens) : 0;
  if (offsets) {  // same rules as the validate-only entry point (reference: kvx_abi.c:161-189)
    const kvx_block_table_t &bt = gather->block_table;
    if (bt.index_dtype != KVX_DTYPE_S32 || (bt.flags & KVX_BLOCK_TABLE_FLAG_KVCACHEINDEX) == 0 ||
        bt.beam_width == 0 || !is_pow2(cache->block_size) ||
        static_cast<uint64_t>(bt.indices_count) !=
            static_cast<uint64_t>(bt.seq_count) * bt.beam_width * 2 * bt.max_blocks_per_seq ||
        bt.indptr != nullptr || bt.indptr_count != 0 || cache->pool.size < sizeof(kvx_pool_desc_t) ||
        cache->pool.bytes_per_block == 0 || cache->pool.primary == nullptr)
      return KVX_STATUS_INVALID_ARGUMENT;
    if (bt.beam_width != 1) return KVX_STATUS_UNSUPPORTED;
    gs.pool[0] = static_cast<const char *>(cache->pool.primary);
    gs.pool[1] = static_cast<const char *>(cache->pool.secondary);
    gs.pool_block_bytes = cache->pool.bytes_per_block;
    gs.beam_width = 1;
  }
  if (ragged) {  // same rules as the validate-only entry point (reference: kvx_abi.c:142-160)
    const kvx_block_table_t &bt = gather->block_table;
    if ((bt.indptr_dtype != KVX_DTYPE_S32 && bt.indptr_dtype != KVX_DTYPE_S64) || bt.beam_width != 1 ||
        bt.indptr == nullptr || bt.indptr_count != bt.seq_count + 1)
      return KVX_STATUS_INVALID_ARGUMENT;
    gs.indptr = bt.indptr;
    gs.indptr64 = bt.indptr_dtype == KVX_DTYPE_S64;
  }

  const cudaStream_t cs = as_stream(stream);
  const DeviceInfo &dev = device_info();

  // ---- vector tier: 16-byte output vectors, each inside one head ------------------------
  const int64_t out_row = H * D * io_elem;
  const int64_t in_vec = fp8 ? 16 / io_elem : 16;  // cache bytes consumed per output vector
  const int64_t chunk_vecs = static_cast<int64_t>(cache->block_size) * (out_row / 16);
  int32_t k_sub = 0, v_sub = 0;
  const bool k_packed = !fp8 && !ragged && view_packed16(gp.k, elem, D, &k_sub);
  const bool v_packed = !fp8 && !ragged && view_packed16(gp.v, elem, D, &v_sub);
  const bool packed = k_packed || v_packed;
  PackedSide k_side{}, v_side{};
  const int64_t tiles_knob = opt(g_opt.packed_tiles);
  const bool tiles = !fp8 && !ragged && !offsets && tiles_knob != 0 &&
                     view_packed_tile(gp.k, elem, D, cache->block_size, &k_side) &&
                     view_packed_tile(gp.v, elem, D, cache->block_size, &v_side);
  const bool vec_ok = !opt(g_opt.force_generic) && (D * io_elem) % 16 == 0 && aligned(gather->io.key.data, 16) &&
                      aligned(gather->io.value.data, 16) &&
                      (tiles || ((k_packed || view_vectorisable(gp.k, elem, D, in_vec)) &&
                                 (v_packed || view_vectorisable(gp.v, elem, D, in_vec)))) &&
                      chunk_vecs < (int64_t{1} << 30) &&
                      S * static_cast<int64_t>(gs.max_blocks) < (int64_t{1} << 31) &&
                      (!offsets || (aligned(gs.pool[0], in_vec) && aligned(gs.pool[1], in_vec) &&
                                    gs.pool_block_bytes % in_vec == 0));
  if (vec_ok && !(ragged && (fp8 || S > 65535))) {
    GatherPagesParams p;
    p.k_base = gp.k.base, p.k_blk = gp.k.blk, p.k_tok = gp.k.tok, p.k_head = gp.k.head;
    p.v_base = gp.v.base, p.v_blk = gp.v.blk, p.v_tok = gp.v.tok, p.v_head = gp.v.head;
    p.k_vec = k_packed ? gp.k.dhi : 16, p.v_vec = v_packed ? gp.v.dhi : 16;
    p.k_sub = k_sub, p.v_sub = v_sub;
    p.key_out = static_cast<char *>(gather->io.key.data);
    p.value_out = static_cast<char *>(gather->io.value.data);
    p.s = gs;
    p.out_row_bytes = out_row;
    p.num_blocks = gp.g.num_blocks;
    p.block_size = gp.g.block_size;
    p.vpr = static_cast<int32_t>(out_row / 16);
    p.vpr_shift = shift_of(p.vpr);
    p.vps = static_cast<int32_t>(D * io_elem / 16);
    p.vps_shift = shift_of(p.vps);
    p.use_prefix = (S <= kMaxPrefixSeqs) ? 1 : 0;
    p.dim = static_cast<int32_t>(D);
    p.ks = ks;
    p.vs = vs;
    if (ragged && !fp8) {
      p.part_vecs = kRaggedTile;  // tokens per CTA
      while (p.part_vecs > 1 && static_cast<int64_t>(p.part_vecs) * (out_row / 16) > 4096) p.part_vecs >>= 1;
      const dim3 rg(static_cast<unsigned>((L + p.part_vecs - 1) / p.part_vecs), static_cast<unsigned>(S));
      {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = rg;
        cfg.blockDim = dim3(kGatherThreads);
        cfg.stream = cs;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = opt(g_opt.pdl) ? 1 : 0;
        if (s32)
          cudaLaunchKernelEx(&cfg, kvx_gather_ragged_kernel<int32_t, 4>, p);
        else
          cudaLaunchKernelEx(&cfg, kvx_gather_ragged_kernel<int64_t, 4>, p);
        return finish_launch();
      }
    }
    if (tiles) {
      // ---- packed pages: transposing tiles.  A tensor in 16-byte groups whose shape allows it is
      // gathered in items of 8 token rows (all heads), any other in items of up to 4 KB of one
      // head's tile; K and V of different kinds take a launch each when the batch is large.
      GatherPackedParams pp;
      pp.g = p;
      pp.k = k_side, pp.v = v_side;
      pp.slots = static_cast<int32_t>(static_cast<int64_t>(cache->block_size) * D * elem / 32);
      pp.head_out_bytes = D * elem;
      const bool rows_shape = tiles_knob != 3 && (D * elem) % 128 == 0 && H * D * elem < (int64_t{1} << 30);
      // item kind per tensor: 1 = rows of 16-byte units, 2 = rows of 2-byte units, 0 = pieces
      auto kind_of = [&](const PackedSide &side) {
        if (!rows_shape) return 0;
        if (side.n_shift == 0 && side.runs % 4 == 0) return 1;
        if (side.n_shift == 3) return 2;
        return 0;
      };
      const int k_kind = kind_of(k_side), v_kind = kind_of(v_side);
      auto launch = [&](int kind, int only) {
        pp.rows = kind, pp.only = only;
        const PackedSide &side = only == 1 ? v_side : k_side;
        pp.span_shift = 0;
        if (kind == 1) {
          pp.pieces = static_cast<int32_t>(D * elem / 128);
          // Few heads (a shard of them): an item of 8 tokens is little per table lookup, so it
          // takes more octets of tokens, up to 16 steps of loads.  (Measured on shards of 1, 2 and
          // 4 heads of 256 bytes: 16 % to 40 % faster than one octet; K and V under one lookup on top
          // of it changed nothing.)
          int lines = side.runs / 4;
          while (lines % 2 == 0 && (H * pp.pieces << (pp.span_shift + 1)) <= 16) lines /= 2, ++pp.span_shift;
          pp.g.parts = lines;
        } else if (kind == 2) {
          pp.g.parts = side.runs;
          pp.pieces = static_cast<int32_t>(D * elem / 128);
        } else {
          pp.pieces = (pp.slots + 127) / 128;
          pp.g.parts = static_cast<int32_t>(H) * pp.pieces;
        }
        const int64_t max_items = S * gs.max_blocks * pp.g.parts * (only < 0 ? 2 : 1);
        pp.g.use_prefix = p.use_prefix && max_items > opt(g_opt.gather_rect_items);
        const int64_t per_sm = std::max<int64_t>(1, opt(g_opt.gather_ctas_per_sm));
        const unsigned ug = static_cast<unsigned>(gather_item_grid(S, gs.max_blocks, pp.g.parts * (only < 0 ? 2 : 1),
                                                                   dev.sm_count, per_sm, kGatherWarps));
        const size_t smem = pp.g.use_prefix ? static_cast<size_t>(S + 1) * sizeof(int32_t) : 0;
#define KVX_GATHER_PACKED(KIND)                                                                       \
  do {                                                                                                \
    if (s32)                                                                                          \
      launch_streaming(kvx_gather_packed_kernel<int32_t, 4, KIND>, ug, kGatherThreads, smem, cs, pp); \
    else                                                                                              \
      launch_streaming(kvx_gather_packed_kernel<int64_t, 4, KIND>, ug, kGatherThreads, smem, cs, pp); \
  } while (0)
        if (kind == 1)
          KVX_GATHER_PACKED(1);
        else if (kind == 2)
          KVX_GATHER_PACKED(2);
        else
          KVX_GATHER_PACKED(0);
#undef KVX_GATHER_PACKED
      };
      const int64_t piece_items = S * gs.max_blocks * H * ((pp.slots + 127) / 128) * 2;
      if (k_kind == v_kind) {
        launch(k_kind, -1);
      } else if (piece_items <= opt(g_opt.gather_rect_items)) {
        launch(0, -1);  // a small batch: one launch of the piece kind for both tensors
      } else {
        launch(k_kind, 0);
        g_launches.fetch_add(1, std::memory_order_relaxed);  // two kernels for this call
        launch(v_kind, 1);
      }
      return finish_launch();
    }
    const bool contiguous_pages = !fp8 && !packed && gp.k.head == D * elem && gp.v.head == D * elem &&
                                  gp.k.tok == H * D * elem && gp.v.tok == H * D * elem;
    const size_t prefix_bytes = p.use_prefix ? static_cast<size_t>(S + 1) * sizeof(int32_t) : 0;

    if (contiguous_pages && opt(g_opt.gather_path) == 1 && !offsets) {
      // ---- bulk tier ----
      BulkParams bp;
      bp.g = p;
      int64_t stage = opt(g_opt.bulk_stage_bytes) / 16 * 16;
      if (stage < 1024) stage = 1024;
      bp.stages = static_cast<int32_t>(opt(g_opt.bulk_stages) < 2 ? 2 : (opt(g_opt.bulk_stages) > kBulkMaxStages ? kBulkMaxStages : opt(g_opt.bulk_stages)));
      bp.pipes = static_cast<int32_t>(opt(g_opt.bulk_pipes) < 1 ? 1 : (opt(g_opt.bulk_pipes) > kBulkMaxPipes ? kBulkMaxPipes : opt(g_opt.bulk_pipes)));
      bp.wait_ns = std::max<int64_t>(1, opt(g_opt.bulk_wait_us)) * 1000;
      bp.test_stall = opt(g_opt.bulk_test_stall) != 0;
      bp.lag = static_cast<int32_t>(opt(g_opt.bulk_lag) < 1 ? 1 : (opt(g_opt.bulk_lag) > bp.stages - 1 ? bp.stages - 1 : opt(g_opt.bulk_lag)));
      const int64_t chunk_bytes = chunk_vecs * 16;
      if (stage > chunk_bytes) stage = chunk_bytes;
      bp.stage_bytes = static_cast<int32_t>(stage);
      bp.g.part_vecs = static_cast<int32_t>(stage / 16);
      bp.g.parts = static_cast<int32_t>((chunk_vecs + bp.g.part_vecs - 1) / bp.g.part_vecs);
      const size_t smem = static_cast<size_t>(bp.pipes) * bp.stages * bp.stage_bytes + prefix_bytes;
      if (smem <= static_cast<size_t>(dev.max_smem_optin) - 1024) {
        const int64_t max_items = S * gs.max_blocks * bp.g.parts * 2;
        int64_t grid = static_cast<int64_t>(dev.sm_count) * (opt(g_opt.bulk_ctas_per_sm) < 1 ? 1 : opt(g_opt.bulk_ctas_per_sm));
        const int64_t need = (max_items + bp.pipes - 1) / bp.pipes;
        if (grid > need) grid = need;
        if (s32) {
          cudaFuncSetAttribute(kvx_gather_bulk_kernel<int32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
          kvx_gather_bulk_kernel<int32_t><<<static_cast<unsigned>(grid), kGatherThreads, smem, cs>>>(bp);
        } else {
          cudaFuncSetAttribute(kvx_gather_bulk_kernel<int64_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
          kvx_gather_bulk_kernel<int64_t><<<static_cast<unsigned>(grid), kGatherThreads, smem, cs>>>(bp);
        }
        return finish_launch();
      }
    }

    // ---- register tier ----
    // The dequantising gather does more work per byte read and measured best with whole pages per
    // warp and a small grid (5 724 GB/s vs 4 886 GB/s with the copy gather's settings).
    int64_t part_vecs = (fp8 ? std::max<int64_t>(opt(g_opt.gather_part_bytes), 32768) : opt(g_opt.gather_part_bytes)) / 16;
    if (part_vecs < 32) part_vecs = 32;
    if (part_vecs > chunk_vecs) part_vecs = chunk_vecs;
    p.part_vecs = static_cast<int32_t>(part_vecs);
    p.parts = static_cast<int32_t>((chunk_vecs + part_vecs - 1) / part_vecs);
    // Grid: see gather_item_grid.
    const int64_t max_items = S * gs.max_blocks * p.parts * 2;
    const int64_t need = (max_items + kGatherWarps - 1) / kGatherWarps;
    // A small rectangle is walked as it is: without the scan a warp asks for its length and its
    // table entry at once, which takes about 1 us off a launch that lasts 25 us (an eighth of
    // the Llama-3-8B batch: 24.4 us instead of 25.5 us), while the items of pages that do not
    // exist cost a resident warp a few cached loads each.  Large rectangles can be mostly
    // padding (decode batches with contexts of 1 to 1 024 pages: 1.8x slower uncompacted).
    if (!fp8 && max_items <= opt(g_opt.gather_rect_items)) p.use_prefix = 0;
    int64_t per_sm = opt(g_opt.gather_ctas_per_sm) < 1 ? 1 : opt(g_opt.gather_ctas_per_sm);
    if (fp8) per_sm = std::min<int64_t>(per_sm, 8);
    int64_t grid = static_cast<int64_t>(dev.sm_count) * per_sm;
    grid = fp8 ? std::max<int64_t>(1, std::min(grid, need))
               : gather_item_grid(S, gs.max_blocks, static_cast<int64_t>(p.parts) * 2, dev.sm_count, per_sm, kGatherWarps);
    const unsigned ug = static_cast<unsigned>(grid);
    if (fp8 && !offsets && io_elem == 2 && opt(g_opt.wide) && (p.vps % 2) == 0 && (p.part_vecs % 2) == 0 &&
        aligned(p.key_out, 32) && aligned(p.value_out, 32) && aligned(p.k_base, 16) && aligned(p.v_base, 16) &&
        p.k_blk % 16 == 0 && p.v_blk % 16 == 0 && p.k_tok % 16 == 0 && p.v_tok % 16 == 0 && p.k_head % 16 == 0 &&
        p.v_head % 16 == 0) {
      // 256-bit stores: 16 cache bytes -> 32 output bytes per lane
      if (io_dtype == KVX_DTYPE_BF16) {
        if (s32)
          launch_streaming(kvx_gather_f8_wide_kernel<BF16, int32_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_f8_wide_kernel<BF16, int64_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);
      } else {
        if (s32)
          launch_streaming(kvx_gather_f8_wide_kernel<F16, int32_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_f8_wide_kernel<F16, int64_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);
      }
      return finish_launch();
    }
    if (fp8) {
#define KVX_F8_GATHER(IoT)                                                                     \
  do {                                                                                         \
    if (offsets)                                                                               \
      launch_streaming(kvx_gather_f8_kernel<IoT, int32_t, 4, true>, ug, kGatherThreads, prefix_bytes, cs, p); \
    else if (s32)                                                                              \
      launch_streaming(kvx_gather_f8_kernel<IoT, int32_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);      \
    else                                                                                       \
      launch_streaming(kvx_gather_f8_kernel<IoT, int64_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);      \
  } while (0)
      if (io_dtype == KVX_DTYPE_BF16)
        KVX_F8_GATHER(BF16);
      else if (io_dtype == KVX_DTYPE_F16)
        KVX_F8_GATHER(F16);
      else
        KVX_F8_GATHER(F32);
#undef KVX_F8_GATHER
      return finish_launch();
    }
    if (offsets) {  // K and V pages are looked up separately; 16-byte vectors, any in-page pitch
      if (contiguous_pages)
        launch_streaming(kvx_gather_pages_kernel<int32_t, false, 8, true>, ug, kGatherThreads, prefix_bytes, cs, p);
      else
        launch_streaming(kvx_gather_pages_kernel<int32_t, true, 8, true>, ug, kGatherThreads, prefix_bytes, cs, p);
      return finish_launch();
    }
    if (opt(g_opt.gather_path) == 2 || packed) {  // warp-granular items
      const bool wide_ok = opt(g_opt.wide) && !packed && (p.part_vecs % 2) == 0 && (p.vpr % 2) == 0 &&
                           aligned(p.k_base, 32) && aligned(p.v_base, 32) && aligned(p.key_out, 32) &&
                           aligned(p.value_out, 32) && p.k_blk % 32 == 0 && p.v_blk % 32 == 0 &&
                           (contiguous_pages || ((p.vps % 2) == 0 && p.k_tok % 32 == 0 && p.v_tok % 32 == 0 &&
                                                 p.k_head % 32 == 0 && p.v_head % 32 == 0));
      if (wide_ok && contiguous_pages) {
        if (s32)
          launch_streaming(kvx_gather_pages_wide_kernel<int32_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_pages_wide_kernel<int64_t, 4>, ug, kGatherThreads, prefix_bytes, cs, p);
        return finish_launch();
      }
      if (wide_ok) {
        if (s32)
          launch_streaming(kvx_gather_pages_wide_kernel<int32_t, 4, true>, ug, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_pages_wide_kernel<int64_t, 4, true>, ug, kGatherThreads, prefix_bytes, cs, p);
        return finish_launch();
      }
      if (s32) {
        if (contiguous_pages)
          launch_streaming(kvx_gather_pages_kernel<int32_t, false, 8>, ug, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_pages_kernel<int32_t, true, 8>, ug, kGatherThreads, prefix_bytes, cs, p);
      } else {
        if (contiguous_pages)
          launch_streaming(kvx_gather_pages_kernel<int64_t, false, 8>, ug, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_pages_kernel<int64_t, true, 8>, ug, kGatherThreads, prefix_bytes, cs, p);
      }
      return finish_launch();
    }
    // CTA-granular items (default): one item = K and V of one part.
    {
      int64_t tile_vecs = opt(g_opt.gather_tile_bytes) / 16;
      if (tile_vecs < kGatherThreads) tile_vecs = kGatherThreads;
      if (tile_vecs > chunk_vecs) tile_vecs = chunk_vecs;
      p.part_vecs = static_cast<int32_t>(tile_vecs);
      p.parts = static_cast<int32_t>((chunk_vecs + tile_vecs - 1) / tile_vecs);
      const int64_t tile_items = S * gs.max_blocks * p.parts;
      int64_t tgrid = static_cast<int64_t>(dev.sm_count) * (opt(g_opt.gather_ctas_per_sm) < 1 ? 1 : opt(g_opt.gather_ctas_per_sm));
      if (tgrid > tile_items) tgrid = tile_items;
      const unsigned tg = static_cast<unsigned>(tgrid);
      if (s32) {
        if (contiguous_pages)
          launch_streaming(kvx_gather_tiles_kernel<int32_t, false, 4>, tg, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_tiles_kernel<int32_t, true, 4>, tg, kGatherThreads, prefix_bytes, cs, p);
      } else {
        if (contiguous_pages)
          launch_streaming(kvx_gather_tiles_kernel<int64_t, false, 4>, tg, kGatherThreads, prefix_bytes, cs, p);
        else
          launch_streaming(kvx_gather_tiles_kernel<int64_t, true, 4>, tg, kGatherThreads, prefix_bytes, cs, p);
      }
      return finish_launch();
    }
  }

  // ---- generic tier ---------------------------------------------------------------------
  if (fp8) {
    if (io_dtype == KVX_DTYPE_BF16) return launch_gather_generic<BF16, F8, true>(gather, gs, gp, cs);
    if (io_dtype == KVX_DTYPE_F16) return launch_gather_generic<F16, F8, true>(gather, gs, gp, cs);
    return launch_gather_generic<F32, F8, true>(gather, gs, gp, cs);
  }
  if (elem == 2) return launch_gather_generic<BF16, BF16, false>(gather, gs, gp, cs);
  return launch_gather_generic<F32, F32, false>(gather, gs, gp, cs);
}

}  // namespace

// ====================================================================== C entry points ==

extern "C" {

KVX_API kvx_status_t kvx_launch_write_kv_f32(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                             void *stream) {
  return write_impl(cache, write, stream, KVX_DTYPE_F32, false, 0);
}
KVX_API kvx_status_t kvx_launch_write_kv_f16(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                             void *stream) {
  return write_impl(cache, write, stream, KVX_DTYPE_F16, false, 0);
}
KVX_API kvx_status_t kvx_launch_write_kv_bf16(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                              void *stream) {
  return write_impl(cache, write, stream, KVX_DTYPE_BF16, false, 0);
}
KVX_API kvx_status_t kvx_launch_write_kv_f8e4m3(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                                void *stream) {
  return write_impl(cache, write, stream, KVX_DTYPE_F8_E4M3, false, 0);
}

KVX_API kvx_status_t kvx_launch_write_kv(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                         void *stream) {
  if (cache == nullptr || write == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype != cache->v.dtype) return KVX_STATUS_INVALID_ARGUMENT;
  switch (cache->k.dtype) {
    case KVX_DTYPE_F16:
    case KVX_DTYPE_BF16:
    case KVX_DTYPE_F32:
    case KVX_DTYPE_F8_E4M3:
      return write_impl(cache, write, stream, cache->k.dtype, false, 0);
    default:
      return KVX_STATUS_UNSUPPORTED;
  }
}

KVX_API kvx_status_t kvx_launch_write_kv_prefill_f32(const kvx_cache_desc_t *cache,
                                                     const kvx_write_desc_t *write, int32_t tokens_per_seq,
                                                     void *stream) {
  return write_impl(cache, write, stream, KVX_DTYPE_F32, true, tokens_per_seq);
}
KVX_API kvx_status_t kvx_launch_write_kv_prefill_f16(const kvx_cache_desc_t *cache,
                                                     const kvx_write_desc_t *write, int32_t tokens_per_seq,
                                                     void *stream) {
  return write_impl(cache, write, stream, KVX_DTYPE_F16, true, tokens_per_seq);
}
KVX_API kvx_status_t kvx_launch_write_kv_prefill_bf16(const kvx_cache_desc_t *cache,
                                                      const kvx_write_desc_t *write, int32_t tokens_per_seq,
                                                      void *stream) {
  return write_impl(cache, write, stream, KVX_DTYPE_BF16, true, tokens_per_seq);
}

KVX_API kvx_status_t kvx_launch_write_kv_prefill(const kvx_cache_desc_t *cache, const kvx_write_desc_t *write,
                                                 int32_t tokens_per_seq, void *stream) {
  if (cache == nullptr || write == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype != cache->v.dtype) return KVX_STATUS_INVALID_ARGUMENT;
  switch (cache->k.dtype) {
    case KVX_DTYPE_F16:
    case KVX_DTYPE_BF16:
    case KVX_DTYPE_F32:
    case KVX_DTYPE_F8_E4M3:
      return write_impl(cache, write, stream, cache->k.dtype, true, tokens_per_seq);
    default:
      return KVX_STATUS_UNSUPPORTED;
  }
}

KVX_API kvx_status_t kvx_launch_gather_kv_f32(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                              void *stream) {
  return gather_impl(cache, gather, nullptr, nullptr, stream, KVX_DTYPE_F32);
}
KVX_API kvx_status_t kvx_launch_gather_kv_f16(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                              void *stream) {
  return gather_impl(cache, gather, nullptr, nullptr, stream, KVX_DTYPE_F16);
}
KVX_API kvx_status_t kvx_launch_gather_kv_bf16(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                               void *stream) {
  return gather_impl(cache, gather, nullptr, nullptr, stream, KVX_DTYPE_BF16);
}
KVX_API kvx_status_t kvx_launch_gather_kv_f8e4m3(const kvx_cache_desc_t *cache,
                                                 const kvx_gather_desc_t *gather,
                                                 const kvx_scale_desc_t *k_scale,
                                                 const kvx_scale_desc_t *v_scale, void *stream) {
  return gather_impl(cache, gather, k_scale, v_scale, stream, KVX_DTYPE_F8_E4M3);
}

KVX_API kvx_status_t kvx_launch_gather_kv(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                          void *stream) {
  if (cache == nullptr || gather == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (cache->k.dtype != cache->v.dtype) return KVX_STATUS_INVALID_ARGUMENT;
  switch (cache->k.dtype) {
    case KVX_DTYPE_F16:
    case KVX_DTYPE_BF16:
    case KVX_DTYPE_F32:
      return gather_impl(cache, gather, nullptr, nullptr, stream, cache->k.dtype);
    default:
      // An fp8 cache needs scales, which a gather descriptor cannot carry: use
      // kvx_launch_gather_kv_f8e4m3.
      return KVX_STATUS_UNSUPPORTED;
  }
}

KVX_API kvx_status_t kvx_launch_gather_kv_varlen(const kvx_cache_desc_t *cache, const kvx_gather_desc_t *gather,
                                                 const void *out_indptr, kvx_dtype_t out_indptr_dtype,
                                                 const kvx_scale_desc_t *k_scale,
                                                 const kvx_scale_desc_t *v_scale, void *stream) {
  if (cache == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  const VarlenOut out{out_indptr, out_indptr_dtype};
  switch (cache->k.dtype) {
    case KVX_DTYPE_F32:
    case KVX_DTYPE_F16:
    case KVX_DTYPE_BF16:
    case KVX_DTYPE_F8_E4M3:
      return gather_impl(cache, gather, k_scale, v_scale, stream, cache->k.dtype, &out);
    default:
      return KVX_STATUS_UNSUPPORTED;
  }
}

KVX_API size_t kvx_kv_scales_workspace_bytes(uint32_t num_kv_heads) {
  const size_t raw = (2 * static_cast<size_t>(num_kv_heads) + 1) * sizeof(uint32_t);
  return (raw + 255) / 256 * 256;
}

// Body of both scale entry points.  `clear_first`: the workspace may hold anything (the shared
// in-library array): the part this call uses is zeroed on the stream once every argument check
// has passed, so a rejected call enqueues nothing at all.
static kvx_status_t kv_scales_impl(const kvx_kv_io_desc_t *io, kvx_scale_granularity_t granularity,
                                   float *k_scale_out, float *v_scale_out, void *workspace,
                                   size_t workspace_bytes, void *stream, bool clear_first) {
  if (io == nullptr || k_scale_out == nullptr || v_scale_out == nullptr || workspace == nullptr)
    return KVX_STATUS_INVALID_ARGUMENT;
  if (io->size < sizeof(kvx_kv_io_desc_t)) return KVX_STATUS_INVALID_ARGUMENT;
  if (granularity != KVX_SCALE_PER_HEAD && granularity != KVX_SCALE_PER_TENSOR) return KVX_STATUS_UNSUPPORTED;
  if (!io_dtype_quantisable(io->key.dtype) || io->value.dtype != io->key.dtype) return KVX_STATUS_UNSUPPORTED;
  if (io->num_kv_heads == 0 || io->head_dim == 0) return KVX_STATUS_INVALID_ARGUMENT;
  const int64_t dims[3] = {io->num_tokens, io->num_kv_heads, io->head_dim};
  kvx_status_t st = check_io_tensor(&io->key, 3, dims);
  if (st != KVX_STATUS_OK) return st;
  st = check_io_tensor(&io->value, 3, dims);
  if (st != KVX_STATUS_OK) return st;
  if (workspace_bytes < kvx_kv_scales_workspace_bytes(io->num_kv_heads) || !aligned(workspace, 256))
    return KVX_STATUS_INVALID_ARGUMENT;
  const int64_t elem = dtype_bytes(io->key.dtype);
  const int64_t T = io->num_tokens, H = io->num_kv_heads, D = io->head_dim;
  if (T > 0 && (io->key.data == nullptr || io->value.data == nullptr)) return KVX_STATUS_INVALID_ARGUMENT;
  // Vector loads need whole 16-byte vectors inside one head.
  if ((D * elem) % 16 != 0 || !aligned(io->key.data, 16) || !aligned(io->value.data, 16) ||
      2 * H * sizeof(uint32_t) > 40960)
    return KVX_STATUS_UNSUPPORTED;

  if (clear_first &&
      cudaMemsetAsync(workspace, 0, kvx_kv_scales_workspace_bytes(io->num_kv_heads), as_stream(stream)) != cudaSuccess) {
    cudaGetLastError();
    return KVX_STATUS_INTERNAL_ERROR;
  }

  ScalesParams p;
  p.key = static_cast<const char *>(io->key.data);
  p.value = static_cast<const char *>(io->value.data);
  p.vpr = static_cast<int32_t>(H * D * elem / 16);
  p.vpr_shift = shift_of(p.vpr);
  p.vps = static_cast<int32_t>(D * elem / 16);
  p.vps_shift = shift_of(p.vps);
  p.total_vecs = T * p.vpr;
  p.heads = static_cast<int32_t>(H);
  int group = 1;
  while (group < 32 && p.vps % (group * 2) == 0) group *= 2;
  p.group = group;
  p.per_tensor = (granularity == KVX_SCALE_PER_TENSOR) ? 1 : 0;
  p.k_out = k_scale_out;
  p.v_out = v_scale_out;
  p.work = static_cast<uint32_t *>(workspace);

  const DeviceInfo &dev = device_info();
  int64_t grid = (p.total_vecs + kScaleThreads * 8 - 1) / (kScaleThreads * 8);
  const int64_t cap = static_cast<int64_t>(dev.sm_count) * 8;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  const size_t smem = 2 * static_cast<size_t>(H) * sizeof(uint32_t);
  const cudaStream_t cs = as_stream(stream);
  // Token rows of a power-of-two number of vectors let every thread keep its place in the row:
  // the grid is then a multiple of the 256-vector blocks of a row.
  const int64_t unit = p.vpr > kScaleThreads ? p.vpr / kScaleThreads : 1;
  const bool fixed = p.vpr_shift >= 0 && p.total_vecs >= 4 * grid * kScaleThreads && grid >= unit;
  if (fixed) grid = grid / unit * unit;
  const unsigned ug = static_cast<unsigned>(grid);
#define KVX_SCALES(IoT)                                                    \
  do {                                                                     \
    if (fixed)                                                             \
      kvx_kv_scales_kernel<IoT, true><<<ug, kScaleThreads, smem, cs>>>(p);  \
    else                                                                   \
      kvx_kv_scales_kernel<IoT, false><<<ug, kScaleThreads, smem, cs>>>(p); \
  } while (0)
  if (io->key.dtype == KVX_DTYPE_BF16)
    KVX_SCALES(BF16);
  else if (io->key.dtype == KVX_DTYPE_F16)
    KVX_SCALES(F16);
  else
    KVX_SCALES(F32);
#undef KVX_SCALES
  return finish_launch();
}

KVX_API kvx_status_t kvx_launch_kv_scales(const kvx_kv_io_desc_t *io, kvx_scale_granularity_t granularity,
                                          float *k_scale_out, float *v_scale_out, void *workspace,
                                          size_t workspace_bytes, void *stream) {
  return kv_scales_impl(io, granularity, k_scale_out, v_scale_out, workspace, workspace_bytes, stream, false);
}

// ---------------------------------------------------------------- scales, no allocation --
// Scratch for kvx_launch_kv_scales_static: the running maxima and the CTA ticket of the scale
// reduction, sized for KVX_KV_SCALES_STATIC_MAX_HEADS heads.  It is part of the loaded module,
// so every device that loads this library holds these 8 448 bytes until the process exits.
constexpr size_t kScalesStaticWords = (2 * KVX_KV_SCALES_STATIC_MAX_HEADS + 1 + 63) / 64 * 64;  // whole 256-byte lines
static __device__ __align__(256) uint32_t g_scales_static_scratch[kScalesStaticWords];

namespace {
// Device address of g_scales_static_scratch per device (NULL = not asked for yet).  In host code
// the array's name is only a handle for the runtime, never an address a kernel may use, so the
// address is asked for once per device, with that device current, and cached.  Two host threads
// that make the first call together both ask and both store the same address.
std::atomic<uint32_t *> g_scales_static_ptr[64];
}  // namespace

KVX_API kvx_status_t kvx_launch_kv_scales_static(const kvx_kv_io_desc_t *io,
                                                 kvx_scale_granularity_t granularity, float *k_scale_out,
                                                 float *v_scale_out, void *stream) {
  if (io == nullptr) return KVX_STATUS_INVALID_ARGUMENT;
  if (io->size < sizeof(kvx_kv_io_desc_t)) return KVX_STATUS_INVALID_ARGUMENT;
  if (io->num_kv_heads > KVX_KV_SCALES_STATIC_MAX_HEADS) return KVX_STATUS_OUT_OF_RANGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KVX_STATUS_INTERNAL_ERROR;
  uint32_t *scratch = g_scales_static_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    void *addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_scales_static_scratch) != cudaSuccess || addr == nullptr) {
      cudaGetLastError();
      return KVX_STATUS_INTERNAL_ERROR;
    }
    scratch = static_cast<uint32_t *>(addr);
    g_scales_static_ptr[dev].store(scratch, std::memory_order_release);
  }
  // The array is shared by every call and keeps whatever the last one left; the reduction needs
  // zeros, so the part it uses is cleared on the caller's stream -- after the argument checks,
  // so that a rejected call leaves the array (which an earlier call may still be using) alone.
  return kv_scales_impl(io, granularity, k_scale_out, v_scale_out, scratch, sizeof(uint32_t) * kScalesStaticWords,
                        stream, true);
}

KVX_API int kvx_b200_device_error(int reset) {
  int word = 0;
  if (cudaMemcpyFromSymbol(&word, g_device_error, sizeof(word)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (word != 0 && reset) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_device_error, &zero, sizeof(zero)) != cudaSuccess) cudaGetLastError();
  }
  return word;
}

KVX_API uint64_t kvx_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
KVX_API void kvx_b200_reset_launch_count(void) { g_launches.store(0, std::memory_order_relaxed); }

KVX_API int kvx_b200_set_option(const char *name, int64_t value) {
  if (name == nullptr) return -1;
  for (const OptionName &o : kOptionNames)
    if (strcmp(o.name, name) == 0) {
      (g_opt.*(o.field)).store(value, std::memory_order_relaxed);
      return 0;
    }
  return -1;
}
KVX_API int64_t kvx_b200_get_option(const char *name) {
  if (name == nullptr) return -1;
  for (const OptionName &o : kOptionNames)
    if (strcmp(o.name, name) == 0) return (g_opt.*(o.field)).load(std::memory_order_relaxed);
  return -1;
}

}  // extern "C"
