// Gather kernels for sm_100a.
//
// Three kernels sum the rows a work item names — a destination row, one segment of a long
// destination row, or one reuse group.  All keep the accumulators in registers and store every
// output row exactly once, so there are no atomics on data and no zero-fill pass (upstream:
// atomicAdd_F per element per part and a torch::zeros per call, reuse_conv_kernel.cu:16-21, 282,
// 303).
//
// gather_rows_kernel ("lanes"): a *lane group* of L threads (L = 4..32, a power of two chosen
// from the feature width) owns one work item.  The group fetches L column entries with one
// coalesced load, broadcasts them with shuffles, and issues U independent 128-bit (64/32-bit
// when alignment forces it) row loads per lane before accumulating, so each warp keeps
// U*C*16 B per lane in flight.  An item's entries are ordered [partial rows | feature rows] so
// each range has one base pointer, the unweighted modes do no multiply, and no load slot is
// issued for an entry that does not exist.  Adds and multiply-adds are the packed f32x2
// instructions of sm_100.
//
// gather_tiles_kernel ("tiles"): for short rows that share many of their entries with their
// neighbours.  One CTA owns a tile of consecutive destination rows, copies the rows used at
// least twice in the tile — partial-sum rows of reuse groups fanned out to these destinations,
// shared feature rows — into shared memory once, and every destination adds them from there;
// only the rows private to a destination are gathered from global memory.
//
// gather_rows_ring_kernel ("ring"): one warp owns one work item and a ring of shared-memory
// stages.  Every gathered row is brought into the ring by one bulk asynchronous copy
// (cp.async.bulk global -> shared, completion counted on an mbarrier per stage; the lane that
// holds a column entry issues that row's copy), and the warp adds rows from shared memory into its
// register accumulators while the copies of the next stages are in flight.  Rows must be
// 16-byte aligned.  Measured about half as fast as the lanes kernel on B200 at every width tried
// — a bulk copy per row of at most a few KB does not keep the copy engine busy — so it only
// runs on request (ROF_KERNEL=ring).  Every wait on an mbarrier is bounded: a wait that runs out
// sets the plan's status word, the warp waits (bounded again) for its copies in flight and
// leaves without storing.
//
// Rows whose work was cut into segments are finished by whichever segment arrives last (a
// per-row arrival counter); it adds the segment sums in slot order, so the result does not
// depend on the arrival order.  split_reduce_kernel does the same as a separate launch for
// callers that issue the phases one by one.
//
// Arithmetic: sum/mean add the gathered values (rounded to nearest); GCN adds
// rsqrt_rn(degrees[src]) * x with one fused multiply-add per term — a single rounding where
// upstream has two (__fmul_rn then add, reuse_conv_kernel.cu:254, 270); the pre-scaled GCN
// mode adds rows that scale_rows_kernel multiplied by rsqrt_rn(degrees[src]) beforehand, which
// is upstream's product bit for bit.  The order of the adds differs from upstream's (arbitrary
// atomic order) in any case.
#include <cstdio>
#include <cstdlib>

#include "rof_internal.h"

namespace rof {
namespace {

template <int VEC>
__device__ __forceinline__ void load_row_vec(float (&v)[VEC], const float* p) {
  if constexpr (VEC == 4) {
    float4 t = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if constexpr (VEC == 2) {
    float2 t = __ldg(reinterpret_cast<const float2*>(p));
    v[0] = t.x; v[1] = t.y;
  } else {
    v[0] = __ldg(p);
  }
}

// L2-coherent load (bypasses L1): for data another SM wrote during this kernel
template <int VEC>
__device__ __forceinline__ void load_row_vec_cg(float (&v)[VEC], const float* p) {
  if constexpr (VEC == 4) {
    float4 t = __ldcg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if constexpr (VEC == 2) {
    float2 t = __ldcg(reinterpret_cast<const float2*>(p));
    v[0] = t.x; v[1] = t.y;
  } else {
    v[0] = __ldcg(p);
  }
}

// plain (coherent) load of data an earlier launch on the same stream wrote
template <int VEC>
__device__ __forceinline__ void load_plain_vec(float (&v)[VEC], const float* p) {
  if constexpr (VEC == 4) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if constexpr (VEC == 2) {
    float2 t = *reinterpret_cast<const float2*>(p);
    v[0] = t.x; v[1] = t.y;
  } else {
    v[0] = *p;
  }
}

template <int VEC>
__device__ __forceinline__ void store_row_vec(float* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  } else {
    *p = v[0];
  }
}

// out = act(r + self_scale * self_x[row][col..] + bias[col..]) for the first `valid` of VEC
// consecutive columns.  The pointers need no alignment: the epilogue reads scalars.
template <int VEC>
__device__ __forceinline__ void apply_epilogue(float (&r)[VEC], const Epilogue& ep, int row, int col, int valid) {
  if (ep.self_x != nullptr) {
    const float* sp = ep.self_x + (int64_t)row * ep.ld_self + col;
#pragma unroll
    for (int t = 0; t < VEC; ++t)
      if (t < valid) r[t] = __fmaf_rn(ep.self_scale, __ldg(sp + t), r[t]);
  }
  if (ep.bias != nullptr) {
#pragma unroll
    for (int t = 0; t < VEC; ++t)
      if (t < valid) r[t] = __fadd_rn(r[t], __ldg(ep.bias + col + t));
  }
  if (ep.relu) {
#pragma unroll
    for (int t = 0; t < VEC; ++t) r[t] = fmaxf(r[t], 0.0f);
  }
}

__device__ __forceinline__ float row_scale(const GatherArgs& a, int row, bool empty) {
  // a row without entries is exactly zero whatever its degree says (upstream never touches it
  // after the zero-fill); 0 * rsqrt(0) would be NaN
  if (empty) return 0.0f;
  if (a.scale_mode == 1) return __frsqrt_rn(__ldg(a.degrees + row));
  if (a.scale_mode == 2) {
    const float d = __ldg(a.degrees + row);
    return (d == 0.0f) ? 0.0f : __frcp_rn(d);
  }
  return 1.0f;
}

// Finishes columns [col0, col0 + VEC) of final output row `row` from the raw sum in r: scale,
// optional add to what an earlier stage stored, epilogue, store (vector store when the output
// allows it, masked scalar stores for a ragged last vector or an unaligned output), mirror.
template <int VEC>
__device__ __forceinline__ void finish_final(const GatherArgs& a, int row, int col0, float (&r)[VEC], float scale) {
  const int valid = min(VEC, a.dim - col0);
  float* op = a.out + (int64_t)(row - a.row_begin) * a.ldo + col0;
  const bool vec_ok = a.out_vec && (valid == VEC || a.out_padded);
#pragma unroll
  for (int t = 0; t < VEC; ++t) r[t] = __fmul_rn(r[t], scale);
  if (a.accumulate) {  // a later stage of a staged pass adds to the row
    if (vec_ok) {
      float p[VEC];
      load_plain_vec<VEC>(p, op);
#pragma unroll
      for (int t = 0; t < VEC; ++t) r[t] = __fadd_rn(p[t], r[t]);
    } else {
#pragma unroll
      for (int t = 0; t < VEC; ++t)
        if (t < valid) r[t] = __fadd_rn(op[t], r[t]);
    }
  }
  apply_epilogue<VEC>(r, a.ep, row, col0, valid);
  if (vec_ok) {
    store_row_vec<VEC>(op, r);
  } else {
#pragma unroll
    for (int t = 0; t < VEC; ++t)
      if (t < valid) op[t] = r[t];
  }
  if (a.mirror != nullptr) {
    const int mrow = a.mirror_ids != nullptr ? __ldg(a.mirror_ids + row) : row;
    float* mp = a.mirror + (int64_t)mrow * a.ldm + col0;
#pragma unroll
    for (int t = 0; t < VEC; ++t)
      if (t < valid) mp[t] = r[t];
  }
}

// The last segment of a split row to arrive sums the row's segment sums in slot order and
// finishes the row.  `sub` / `nsub`: this thread's index among the `nsub` threads that share
// the work (they cover vectors sub, sub + nsub, ...).
template <int VEC>
__device__ __forceinline__ void reduce_split_row(const GatherArgs& a, const SplitRow sr, int sub, int nsub) {
  const int nvec = (a.dim + VEC - 1) / VEC;
  const float scale = row_scale(a, sr.row, false);
  for (int iv = sub; iv < nvec; iv += nsub) {
    float s[VEC];
#pragma unroll
    for (int t = 0; t < VEC; ++t) s[t] = 0.0f;
    const float* sp = a.slots + (int64_t)sr.first_slot * a.lds + (int64_t)iv * VEC;
    for (int k = 0; k < sr.count; ++k) {
      float v[VEC];
      load_row_vec_cg<VEC>(v, sp + (int64_t)k * a.lds);
#pragma unroll
      for (int t = 0; t < VEC; ++t) s[t] = __fadd_rn(s[t], v[t]);
    }
    finish_final<VEC>(a, sr.row, iv * VEC, s, scale);
  }
}

// acc += v and acc += w * v on VEC consecutive floats.  Pairs of floats go through the packed
// f32x2 instructions of sm_100 (one instruction per two adds; each half rounds like the scalar
// instruction, so results do not change).
template <int VEC>
__device__ __forceinline__ void acc_add(float (&acc)[VEC], const float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    acc[0] = __fadd_rn(acc[0], v[0]);
  } else {
#pragma unroll
    for (int t = 0; t < VEC; t += 2) {
      const float2 r = __fadd2_rn(make_float2(acc[t], acc[t + 1]), make_float2(v[t], v[t + 1]));
      acc[t] = r.x; acc[t + 1] = r.y;
    }
  }
}

template <int VEC>
__device__ __forceinline__ void acc_fma(float (&acc)[VEC], float w, const float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    acc[0] = __fmaf_rn(w, v[0], acc[0]);
  } else {
#pragma unroll
    for (int t = 0; t < VEC; t += 2) {
      const float2 r = __ffma2_rn(make_float2(w, w), make_float2(v[t], v[t + 1]), make_float2(acc[t], acc[t + 1]));
      acc[t] = r.x; acc[t + 1] = r.y;
    }
  }
}

// Where the rows of one range of entries live.  Plain: every entry c names row (c - c_offset)
// of one buffer.  MIXED (tile kernel): entries >= num_nodes name partial rows, the others feature
// rows, selected per entry.  Pointers already include this lane's column offset.
struct RowSource {
  const float* base; int64_t ld; int c_offset;      // plain
  const float* partials; int64_t ldp; int num_nodes;  // MIXED only
};

// Loads UU rows — entries j .. j+UU-1 of the window of L entries the group holds in `c` (and
// their weights in `w`) — and adds them to acc.  No per-entry predicate: the caller only asks for
// entries that exist.
template <int VEC, int L, int C, int UU, bool WEIGHTED, bool MIXED>
__device__ __forceinline__ void gather_batch(float (&acc)[C][VEC], int c, float w, int j, const RowSource& src,
                                             unsigned gmask, const bool (&active)[C]) {
  float v[UU][C][VEC];
#pragma unroll
  for (int u = 0; u < UU; ++u) {
    const int cj = __shfl_sync(gmask, c, j + u, L);
    const float* rp;
    if constexpr (MIXED)
      rp = (cj >= src.num_nodes) ? src.partials + (int64_t)(cj - src.num_nodes) * src.ldp : src.base + (int64_t)cj * src.ld;
    else
      rp = src.base + (int64_t)cj * src.ld;
#pragma unroll
    for (int k = 0; k < C; ++k) {
      if (active[k]) {
        load_row_vec<VEC>(v[u][k], rp + k * (L * VEC));
      } else {
#pragma unroll
        for (int t = 0; t < VEC; ++t) v[u][k][t] = 0.0f;
      }
    }
  }
#pragma unroll
  for (int u = 0; u < UU; ++u) {
    if constexpr (WEIGHTED) {
      const float wj = __shfl_sync(gmask, w, j + u, L);
#pragma unroll
      for (int k = 0; k < C; ++k) acc_fma<VEC>(acc[k], wj, v[u][k]);
    } else {
#pragma unroll
      for (int k = 0; k < C; ++k) acc_add<VEC>(acc[k], v[u][k]);
    }
  }
}

// One window of a range: the group's lanes fetch up to L consecutive column entries (and, for GCN,
// the weight of each feature row); lane l holds entry e + l.
template <int L, bool WEIGHTED, bool MIXED>
__device__ __forceinline__ void load_window(const int32_t* __restrict__ col, int e, int end, const RowSource& src,
                                            const float* __restrict__ degrees, int lane, int& c, float& w) {
  const int mine = e + lane;
  c = 0;
  w = 1.0f;
  if (mine < end) {
    c = __ldg(col + mine);
    if constexpr (WEIGHTED) {
      if (!MIXED || c < src.num_nodes) w = __frsqrt_rn(__ldg(degrees + c));
    }
    if constexpr (!MIXED) c -= src.c_offset;
  }
}

// Adds the rows of the first `cnt` entries of a window in batches of U; what is left is walked in
// batches of 4, 2 and 1, so that no load slot is issued for an entry that does not exist (short
// rows are bound by instruction issue as much as by latency).
template <int VEC, int L, int C, int U, bool WEIGHTED, bool MIXED>
__device__ __forceinline__ void consume_window(float (&acc)[C][VEC], int c, float w, int cnt, const RowSource& src,
                                               int lane, unsigned gmask, const bool (&active)[C]) {
  int j = 0;
  for (; j + U <= cnt; j += U) gather_batch<VEC, L, C, U, WEIGHTED, MIXED>(acc, c, w, j, src, gmask, active);
  if constexpr (U > 4) {
    if (cnt - j >= 4) { gather_batch<VEC, L, C, 4, WEIGHTED, MIXED>(acc, c, w, j, src, gmask, active); j += 4; }
  }
  if constexpr (U > 2) {
    if (cnt - j >= 2) { gather_batch<VEC, L, C, 2, WEIGHTED, MIXED>(acc, c, w, j, src, gmask, active); j += 2; }
  }
  if constexpr (U > 1) {
    if (cnt - j >= 1) gather_batch<VEC, L, C, 1, WEIGHTED, MIXED>(acc, c, w, j, src, gmask, active);
  }
}

// acc += sum over col[begin, end) of (WEIGHTED ? rsqrt(degrees[c]) : 1) * row(c), window by window.
template <int VEC, int L, int C, int U, bool WEIGHTED, bool MIXED>
__device__ __forceinline__ void accumulate_range(float (&acc)[C][VEC], const int32_t* __restrict__ col, int begin,
                                                 int end, const RowSource& src, const float* __restrict__ degrees,
                                                 int lane, unsigned gmask, const bool (&active)[C]) {
  for (int e = begin; e < end; e += L) {
    int c;
    float w;
    load_window<L, WEIGHTED, MIXED>(col, e, end, src, degrees, lane, c, w);
    consume_window<VEC, L, C, U, WEIGHTED, MIXED>(acc, c, w, min(L, end - e), src, lane, gmask, active);
  }
}

// Counts a stored segment in on its row's arrival counter; the last segment to arrive adds the
// row's segment sums in slot order and finishes the row.  Cold path, kept out of line so that
// it does not cost the gather loops registers.  `leader` is the one thread of the item's group
// that touches the counter, `gmask` the group's lanes, `writer` whether this thread holds
// vectors (sub, sub + nsub, ...) of the row.
template <int VEC>
__device__ __noinline__ void segment_arrived(const GatherArgs& a, int slot, bool writer, int sub, int nsub,
                                             bool leader, unsigned gmask, int leader_lane) {
  __threadfence();                  // this thread's part of the slot is visible device-wide ...
  __syncwarp(gmask);                // ... before the group's leader counts the segment in
  const int owner = __ldg(a.slot_owner + slot);
  const int4 raw = __ldg(reinterpret_cast<const int4*>(a.split) + owner);
  int last = 0;
  if (leader) {
    const int seen = atomicAdd(a.arrive + owner, 1);
    last = (seen == raw.z - 1);
    if (last) a.arrive[owner] = 0;  // ready for the next pass; nobody else touches it any more
  }
  last = __shfl_sync(gmask, last, leader_lane);
  if (!last) return;
  __threadfence();
  if (writer) reduce_split_row<VEC>(a, SplitRow{raw.x, raw.y, raw.z, 0}, sub, nsub);
}

// Stores the raw sum of a segment into its scratch slot, then — when the plan carries arrival
// counters — counts the segment in (segment_arrived).
template <int VEC, int C>
__device__ __forceinline__ void finish_segment(const GatherArgs& a, int slot, float (&acc)[C][VEC],
                                               const bool (&active)[C], bool writer, int sub, int nsub, bool leader,
                                               unsigned gmask, int leader_lane) {
  if (writer) {
    float* op = a.slots + (int64_t)slot * a.lds;
#pragma unroll
    for (int k = 0; k < C; ++k)
      if (active[k]) store_row_vec<VEC>(op + (int64_t)(sub + k * nsub) * VEC, acc[k]);
  }
  if (a.arrive != nullptr) segment_arrived<VEC>(a, slot, writer, sub, nsub, leader, gmask, leader_lane);
}

// VEC floats per load, L lanes per item, C vectors per lane (L*C*VEC >= dim), U rows in flight;
// WEIGHTED: multiply each feature row by rsqrt(degrees[col]) (GCN).
template <int VEC, int L, int C, int U, bool WEIGHTED>
__global__ void __launch_bounds__(256, (C <= 2 ? 4 : (C * U <= 6 ? 3 : (C * U <= 12 ? 2 : 1)))) gather_rows_kernel(const __grid_constant__ GatherArgs a) {
  static_assert(U <= L && (L % U) == 0, "a batch of L entries is a whole number of unrolled steps");
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int item_id = (int)(gtid / L);
  if (item_id >= a.num_items) return;  // whole lane groups leave together
  const int lane = threadIdx.x & (L - 1);
  const int group_lane0 = (threadIdx.x & 31) & ~(L - 1);
  const unsigned gmask = (L == 32) ? 0xffffffffu : (((1u << L) - 1u) << group_lane0);

  const int4 raw = __ldg(reinterpret_cast<const int4*>(a.items) + item_id);
  const int begin = raw.x, end = raw.y, dst = raw.z, mid = raw.w;  // [begin,mid) partial rows, [mid,end) feature rows
  const int nvec = (a.dim + VEC - 1) / VEC;

  bool active[C];
  float acc[C][VEC];
#pragma unroll
  for (int k = 0; k < C; ++k) {
    active[k] = (lane + k * L) < nvec;
#pragma unroll
    for (int t = 0; t < VEC; ++t) acc[k][t] = 0.0f;
  }

  if (mid > begin) {
    const RowSource src{a.partials + lane * VEC, a.ldp, a.num_nodes, nullptr, 0, 0};
    accumulate_range<VEC, L, C, U, false, false>(acc, a.col, begin, mid, src, nullptr, lane, gmask, active);
  }
  if (end > mid) {
    const RowSource src{a.x + lane * VEC, a.ldx, 0, nullptr, 0, 0};
    accumulate_range<VEC, L, C, U, WEIGHTED, false>(acc, a.col, mid, end, src, a.degrees, lane, gmask, active);
  }

  if (dst >= 0) {
    const float scale = row_scale(a, dst, begin == end);
#pragma unroll
    for (int k = 0; k < C; ++k)
      if (active[k]) finish_final<VEC>(a, dst, (lane + k * L) * VEC, acc[k], scale);
    if (a.mirror != nullptr && a.mirror_flag_col >= 0 && lane == 0)
      a.mirror[(int64_t)(a.mirror_ids != nullptr ? __ldg(a.mirror_ids + dst) : dst) * a.ldm + a.mirror_flag_col] = 1.0f;
  } else {
    finish_segment<VEC, C>(a, -dst - 1, acc, active, true, lane, L, lane == 0, gmask, group_lane0);
  }
}

// ---------------------------------------------------------------------------------------
// ring kernel: bulk asynchronous copies into a shared-memory ring
// ---------------------------------------------------------------------------------------
constexpr uint32_t kWaitPolls = 1u << 20;      // polls of about a microsecond each ...
constexpr long long kWaitCycles = 2000000000;  // ... and never more than about a second of SM clocks

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One poll: may suspend the thread for up to about `hint_ns` while the phase is incomplete.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}

// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity, 1000)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 0; i < kWaitPolls; ++i) {
    if (mbar_try_wait(bar, parity, 1000)) return true;
    if ((i & 255u) == 255u && clock64() - t0 > kWaitCycles) return false;
  }
  return false;
}

// One row: global -> this CTA's shared memory, completion counted in bytes on `bar`.  Both
// addresses 16-byte aligned, `bytes` a multiple of 16.  No multicast, local memory only.
__device__ __forceinline__ void bulk_row_to_smem(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

struct RingCfg {
  int stage_rows;   // B: rows per stage, a power of two <= 32
  int log_stages;   // S = 1 << log_stages stages per warp
  int row_bytes;    // bytes copied per row (a multiple of 16)
};

// C float4 per lane per row, R rows consumed side by side (32 / R lanes per row; R > 1 only
// with C == 1, for rows of at most 16 vectors).
template <int C, int R>
__global__ void __launch_bounds__(256) gather_rows_ring_kernel(const __grid_constant__ GatherArgs a, const RingCfg cfg) {
  constexpr int LPR = 32 / R;
  extern __shared__ __align__(128) unsigned char ring_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int item_id = blockIdx.x * warps + warp;
  if (item_id >= a.num_items) return;  // whole warps leave together; nothing below syncs the block
  const int B = cfg.stage_rows, S = 1 << cfg.log_stages;
  const uint32_t rb = (uint32_t)cfg.row_bytes;
  const uint32_t stage_bytes = (uint32_t)B * rb;
  const unsigned char* ring = ring_smem + (size_t)warp * S * stage_bytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t bar0 = smem_u32(ring_smem + (size_t)warps * S * stage_bytes) + (uint32_t)(warp * S * 8);
  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(bar0 + 8u * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  const int4 raw = __ldg(reinterpret_cast<const int4*>(a.items) + item_id);
  const int begin = raw.x, dst = raw.z;
  const int n = raw.y - raw.x;
  const int nb = (n + B - 1) / B;
  const int sr = lane / LPR, vi = lane % LPR;
  const int nvec = (a.dim + 3) >> 2;

  bool active[C];
  float acc[C][4];
#pragma unroll
  for (int k = 0; k < C; ++k) {
    active[k] = (vi + k * LPR) < nvec;
#pragma unroll
    for (int t = 0; t < 4; ++t) acc[k][t] = 0.0f;
  }

  // column entries: this lane holds entry 32*win + lane of the item, and the one 32 further on
  const int32_t* cp = a.col + begin;
  int cw = (lane < n) ? __ldg(cp + lane) : 0;
  int cw_next = (32 + lane < n) ? __ldg(cp + 32 + lane) : 0;
  int win = 0;

  auto produce = [&](int b) {
    const int e0 = b * B;
    if ((e0 >> 5) != win) {
      win = e0 >> 5;
      cw = cw_next;
      const int nx = (win + 1) * 32 + lane;
      cw_next = (nx < n) ? __ldg(cp + nx) : 0;
    }
    const int cnt = min(B, n - e0);
    const int c = __shfl_sync(0xffffffffu, cw, ((e0 & 31) + lane) & 31);
    const int s = b & (S - 1);
    const uint32_t bar = bar0 + 8u * s;
    if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)cnt * rb);
    if (lane < cnt) {
      const float* src = (c >= a.num_nodes) ? a.partials + (int64_t)(c - a.num_nodes) * a.ldp
                                            : a.x + (int64_t)c * a.ldx;
      bulk_row_to_smem(ring_u32 + (uint32_t)s * stage_bytes + (uint32_t)lane * rb, src, rb, bar);
    }
  };

  const int ahead = min(S, nb);
  for (int b = 0; b < ahead; ++b) produce(b);

  int failed_at = -1;
  for (int b = 0; b < nb; ++b) {
    const int s = b & (S - 1);
    if (!mbar_wait(bar0 + 8u * s, (uint32_t)(b >> cfg.log_stages) & 1u)) {
      failed_at = b;
      break;
    }
    const int cnt = min(B, n - b * B);
    const unsigned char* stage = ring + (size_t)s * stage_bytes + (size_t)vi * 16;
#pragma unroll 4
    for (int j0 = 0; j0 < cnt; j0 += R) {
      const int j = j0 + sr;
      if (R == 1 || j < cnt) {
        const unsigned char* rp = stage + (size_t)j * rb;
#pragma unroll
        for (int k = 0; k < C; ++k) {
          if (active[k]) {
            const float4 v4 = *reinterpret_cast<const float4*>(rp + (size_t)k * (LPR * 16));
            const float v[4] = {v4.x, v4.y, v4.z, v4.w};
            acc_add<4>(acc[k], v);
          }
        }
      }
    }
    __syncwarp();  // every lane has read the stage before its next copies are issued
    if (b + S < nb) produce(b + S);
  }
  if (failed_at >= 0) {
    // Report, then give the copies still in flight a second bounded chance to land so that
    // nothing writes into this shared memory after the block has gone.
    if (lane == 0 && a.status != nullptr) atomicExch(a.status, 1);
    const int issued = min(nb, failed_at + S);
    for (int b = failed_at; b < issued; ++b)
      (void)mbar_wait(bar0 + 8u * (b & (S - 1)), (uint32_t)(b >> cfg.log_stages) & 1u);
    return;
  }

  if (R > 1) {  // the R partial sums of the same columns sit LPR lanes apart
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1)
#pragma unroll
      for (int t = 0; t < 4; ++t) acc[0][t] = __fadd_rn(acc[0][t], __shfl_xor_sync(0xffffffffu, acc[0][t], off));
  }
  if (dst >= 0) {
    if (sr == 0) {
      const float scale = row_scale(a, dst, n == 0);
#pragma unroll
      for (int k = 0; k < C; ++k)
        if (active[k]) finish_final<4>(a, dst, (vi + k * LPR) * 4, acc[k], scale);
      if (a.mirror != nullptr && a.mirror_flag_col >= 0 && lane == 0)
        a.mirror[(int64_t)(a.mirror_ids != nullptr ? __ldg(a.mirror_ids + dst) : dst) * a.ldm + a.mirror_flag_col] = 1.0f;
    }
  } else {
    finish_segment<4, C>(a, -dst - 1, acc, active, sr == 0, vi, LPR, lane == 0, 0xffffffffu, 0);
  }
}

// ---------------------------------------------------------------------------------------
// tile kernel: rows that neighbouring destinations share are staged once in shared memory
// ---------------------------------------------------------------------------------------
// One CTA owns one tile of up to kTileRows short destination rows.  The plan lists the entries
// that occur at least twice in the tile (partial-sum rows of reuse groups fanned out to these
// destinations, feature rows several of them gather); the CTA copies those rows into shared
// memory once (weighted by rsqrt(degrees) in GCN mode, so the adds below need no multiply), and
// each lane group then sums its destination from [slots in shared memory | rows in global
// memory].  A destination whose neighbours are mostly shared issues one round of global loads
// instead of four or five; short rows are bound by those dependent rounds and by instruction issue,
// not by bandwidth.
// Upstream stages one part's partial sum per warp in shared memory and fans it out with atomics
// (reuse_conv_kernel.cu:902-952); here a tile's destinations read every shared row from the
// same copy and each output row is still stored exactly once.
template <int L, int C, int U, bool WEIGHTED>
__global__ void __launch_bounds__(256, (C <= 2 ? 4 : 2)) gather_tiles_kernel(const __grid_constant__ GatherArgs a,
                                                                             const TileArgs t) {
  extern __shared__ __align__(16) float4 tile_smem[];
  constexpr int G = 256 / L;                       // lane groups per CTA
  const int lane = threadIdx.x & (L - 1);
  const int group = threadIdx.x / L;
  const int group_lane0 = (threadIdx.x & 31) & ~(L - 1);
  const unsigned gmask = (L == 32) ? 0xffffffffu : (((1u << L) - 1u) << group_lane0);
  const int nvec = (a.dim + 3) >> 2;
  const int rowvec = L * C;                        // float4 per staged row (>= nvec)

  const int4 td = __ldg(reinterpret_cast<const int4*>(t.tiles) + blockIdx.x);
  const int first_item = td.x, num_items = td.y, stage_begin = td.z, stage_count = td.w;

  bool active[C];
#pragma unroll
  for (int k = 0; k < C; ++k) active[k] = (lane + k * L) < nvec;

  const RowSource gsrc{a.x + lane * 4, a.ldx, 0, a.partials + lane * 4, a.ldp, a.num_nodes};

  // this group's first item: fetched before the staging so that both latencies overlap
  int4 raw = make_int4(0, 0, 0, 0);
  if (group < num_items) raw = __ldg(reinterpret_cast<const int4*>(t.titems) + first_item + group);

  // phase 1: stage the tile's shared rows (weighted for GCN, so that the adds below need no multiply).
  // Gathering the first item's private rows while the staged rows are on their way was tried and
  // measured no faster (community graph, width 64: 0.67 vs 0.66 ms).
#pragma unroll 2
  for (int s = group; s < stage_count; s += G) {
    const int c = __ldg(t.stage_col + stage_begin + s);
    const float* rp;
    float w = 1.0f;
    if (c >= a.num_nodes) {
      rp = a.partials + (int64_t)(c - a.num_nodes) * a.ldp;
    } else {
      rp = a.x + (int64_t)c * a.ldx;
      if constexpr (WEIGHTED) w = __frsqrt_rn(__ldg(a.degrees + c));
    }
#pragma unroll
    for (int k = 0; k < C; ++k) {
      if (active[k]) {
        float4 v = __ldg(reinterpret_cast<const float4*>(rp) + lane + k * L);
        if constexpr (WEIGHTED) {
          v.x = __fmul_rn(w, v.x); v.y = __fmul_rn(w, v.y); v.z = __fmul_rn(w, v.z); v.w = __fmul_rn(w, v.w);
        }
        tile_smem[s * rowvec + lane + k * L] = v;
      }
    }
  }
  __syncthreads();

  // phase 2: one lane group per destination row
  for (int it = group; it < num_items; it += G) {
    const int begin = raw.x, end = raw.y, dst = raw.z, mid = raw.w;   // [begin,mid) slots, [mid,end) global rows
    if (it + G < num_items) raw = __ldg(reinterpret_cast<const int4*>(t.titems) + first_item + it + G);
    float acc[C][4];
#pragma unroll
    for (int k = 0; k < C; ++k)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[k][q] = 0.0f;
    // rows read from global memory (partial rows and feature rows, selected per entry)
    if (end > mid)
      accumulate_range<4, L, C, U, WEIGHTED, true>(acc, t.tcol, mid, end, gsrc, a.degrees, lane, gmask, active);
    // rows staged in shared memory
    for (int e = begin; e < mid; e += L) {
      const int mine = e + lane;
      const int sl = (mine < mid) ? __ldg(t.tcol + mine) : 0;
      const int cnt = min(L, mid - e);
      for (int j = 0; j < cnt; ++j) {
        const int sj = __shfl_sync(gmask, sl, j, L);
#pragma unroll
        for (int k = 0; k < C; ++k) {
          if (active[k]) {
            const float4 v4 = tile_smem[sj * rowvec + lane + k * L];
            const float v[4] = {v4.x, v4.y, v4.z, v4.w};
            acc_add<4>(acc[k], v);
          }
        }
      }
    }
    const float scale = row_scale(a, dst, begin == end);
#pragma unroll
    for (int k = 0; k < C; ++k)
      if (active[k]) finish_final<4>(a, dst, (lane + k * L) * 4, acc[k], scale);
  }
}

// out[row] = scale * sum of the row's segment sums, added in segment order (deterministic).
__global__ void __launch_bounds__(256) split_reduce_kernel(const ReduceArgs a) {
  const int warp = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  if (warp >= a.num_rows) return;
  const int lane = threadIdx.x & 31;
  const int4 raw = __ldg(reinterpret_cast<const int4*>(a.rows) + warp);
  const int row = raw.x, first = raw.y, count = raw.z;
  float scale = 1.0f;
  if (a.scale_mode == 1) {
    scale = __frsqrt_rn(__ldg(a.degrees + row));
  } else if (a.scale_mode == 2) {
    const float d = __ldg(a.degrees + row);
    scale = (d == 0.0f) ? 0.0f : __frcp_rn(d);
  }
  float* op = a.out + (int64_t)(row - a.row_begin) * a.ldo;
  for (int d = lane; d < a.dim; d += 32) {
    float s = 0.0f;
    for (int k = 0; k < count; ++k) s = __fadd_rn(s, a.slots[(int64_t)(first + k) * a.lds + d]);
    float r[1] = {__fmul_rn(s, scale)};
    if (a.accumulate) r[0] = __fadd_rn(op[d], r[0]);
    apply_epilogue<1>(r, a.ep, row, d, 1);
    op[d] = r[0];
  }
}

// out[r][0:dim] = f(degrees[r]) * x[r][0:dim]; columns [dim, pad_to) of out are set to zero.
// op 0: f = 1 (copy into a padded buffer), 1: rsqrt, 2: reciprocal (0 for degree 0).
__global__ void __launch_bounds__(256) scale_rows_kernel(const float* __restrict__ x, int64_t ldx,
                                                         const float* __restrict__ degrees, float* __restrict__ out,
                                                         int64_t ldo, int num_rows, int dim, int pad_to, int op) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp0; r < num_rows; r += nwarps) {
    float f = 1.0f;
    if (op == 1) {
      f = __frsqrt_rn(__ldg(degrees + r));
    } else if (op == 2) {
      const float d = __ldg(degrees + r);
      f = (d == 0.0f) ? 0.0f : __frcp_rn(d);
    }
    const float* xp = x + r * ldx;
    float* op_ = out + r * ldo;
    for (int d = lane; d < pad_to; d += 32) op_[d] = (d < dim) ? __fmul_rn(f, xp[d]) : 0.0f;
  }
}

// Streams `n` float4 `repeats` times through L2-only loads and keeps the sum alive: a plain
// bandwidth probe (L2 when the buffer fits it, HBM when it does not).
__global__ void __launch_bounds__(256) probe_read_kernel(const float4* __restrict__ buf, int64_t n, int repeats,
                                                         float* __restrict__ sink) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < repeats; ++r) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < n; i += 4 * stride) {
      const float4 v0 = __ldcg(buf + i), v1 = __ldcg(buf + i + stride), v2 = __ldcg(buf + i + 2 * stride),
                   v3 = __ldcg(buf + i + 3 * stride);
      s.x += v0.x + v1.x + v2.x + v3.x; s.y += v0.y + v1.y + v2.y + v3.y;
      s.z += v0.z + v1.z + v2.z + v3.z; s.w += v0.w + v1.w + v2.w + v3.w;
    }
    for (; i < n; i += stride) {
      const float4 v = __ldcg(buf + i);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
  }
  const float t = s.x + s.y + s.z + s.w;
  if (t == 1.2345e-30f) *sink = t;  // never true for the probe's data; keeps the loads
}

template <int VEC, int L, int C, int U>
cudaError_t launch_one(const GatherArgs& a, cudaStream_t stream) {
  const int threads = 256;
  const int64_t total = (int64_t)a.num_items * L;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  if (a.weight_gcn)
    gather_rows_kernel<VEC, L, C, U, true><<<(unsigned)blocks, threads, 0, stream>>>(a);
  else
    gather_rows_kernel<VEC, L, C, U, false><<<(unsigned)blocks, threads, 0, stream>>>(a);
  return cudaGetLastError();
}

// Rows of 17..32 vectors run on 16 lanes with two vectors per lane instead of a whole warp with
// one: two items per warp halve what every item pays once (descriptor, column entries, shuffles,
// the store) for the same bytes per load — measured on B200 at widths 100 and 128: 5-9 % faster on
// rows of ~490 entries, 5-11 % at ~50, 18-22 % at 14-21.  Rows of 9..16 vectors gain from the same
// step (8 lanes, two vectors) only when the items are very short (the reuse groups of phase A,
// part_size entries each: 4 % of a pass); at 14 or 50 entries per row it loses 10-15 %.
// ROF_SHORT_ROWS = 0 | 1 forces the old / the new shapes everywhere (experiments, tests).
constexpr int kShortItemEntries = 6;

static int lane_shape_override() {
  const char* e = std::getenv("ROF_SHORT_ROWS");
  return e == nullptr ? -1 : (e[0] == '1' ? 1 : 0);
}

template <int VEC>
cudaError_t dispatch_width(const GatherArgs& a, cudaStream_t stream) {
  const int nvec = (a.dim + VEC - 1) / VEC;
  if (nvec <= 4) return launch_one<VEC, 4, 1, 4>(a, stream);
  if (nvec <= 8) return launch_one<VEC, 8, 1, 8>(a, stream);
  if constexpr (VEC == 4) {
    const int force = lane_shape_override();
    if (nvec > 16 && nvec <= 32 && force != 0) return launch_one<VEC, 16, 2, 4>(a, stream);
    if (nvec <= 16 && (force == 1 || (force < 0 && a.entries_per_item > 0 && a.entries_per_item <= kShortItemEntries)))
      return launch_one<VEC, 8, 2, 4>(a, stream);
  }
  if (nvec <= 16) return launch_one<VEC, 16, 1, 8>(a, stream);
  const int c = (nvec + 31) / 32;
  // wide rows (measured on B200, 114.6M-edge graph): 3 vectors per lane run best with two rows in
  // flight, 4 to 6 with one row in flight and three blocks per SM (width 602: 15.2 vs 18.8 ms)
  switch (c) {
    case 1: return launch_one<VEC, 32, 1, 8>(a, stream);
    case 2: return launch_one<VEC, 32, 2, 4>(a, stream);
    case 3: return launch_one<VEC, 32, 3, 2>(a, stream);
    case 4: return launch_one<VEC, 32, 4, 1>(a, stream);
    case 5: return launch_one<VEC, 32, 5, 1>(a, stream);
    case 6: return launch_one<VEC, 32, 6, 1>(a, stream);
    case 7: case 8: return launch_one<VEC, 32, 8, 1>(a, stream);
    case 9: case 10: return launch_one<VEC, 32, 10, 1>(a, stream);
    case 11: case 12: return launch_one<VEC, 32, 12, 1>(a, stream);
    default: return launch_one<VEC, 32, 16, 1>(a, stream);
  }
}

inline bool aligned_to(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

inline int64_t round_up_to(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// ---- ring launch ------------------------------------------------------------------------
constexpr int kRingMaxSmem = 200 * 1024;   // per block; the SM has 227 KB for one block

struct RingChoice {
  RingCfg cfg;
  int warps;
  size_t smem;
};

// Stage shape for rows of `row_bytes`: about 4 KB per stage, four stages per warp, and as many
// warps per block as leave room for two blocks per SM.  ROF_RING="rows,stages,warps" overrides
// (experiments).
RingChoice choose_ring(int row_bytes) {
  int rows = 1;
  while (rows < 32 && rows * 2 * row_bytes <= 4096) rows *= 2;
  int log_stages = 2, warps = 8;
  if (const char* e = std::getenv("ROF_RING")) {
    int r = 0, s = 0, w = 0;
    if (std::sscanf(e, "%d,%d,%d", &r, &s, &w) == 3 && r >= 1 && r <= 32 && (r & (r - 1)) == 0 && s >= 1 && s <= 32 &&
        (s & (s - 1)) == 0 && w >= 1 && w <= 8) {
      rows = r; warps = w; log_stages = 0;
      while ((1 << log_stages) < s) ++log_stages;
    }
  }
  RingChoice c;
  c.cfg = RingCfg{rows, log_stages, row_bytes};
  c.warps = warps;
  auto bytes = [&](int w) { return (size_t)w * (1u << c.cfg.log_stages) * ((size_t)rows * row_bytes + 8); };
  while (c.warps > 1 && bytes(c.warps) > (size_t)kRingMaxSmem / 2) c.warps /= 2;
  while (c.cfg.log_stages > 0 && bytes(c.warps) > (size_t)kRingMaxSmem) --c.cfg.log_stages;
  c.smem = bytes(c.warps);
  return c;
}

template <int C, int R>
cudaError_t launch_ring_one(const GatherArgs& a, const RingChoice& rc, cudaStream_t stream) {
  // the opt-in to more than 48 KB of dynamic shared memory is per device
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t ge = cudaGetDevice(&dev);
  if (ge != cudaSuccess) return ge;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    ge = cudaFuncSetAttribute(gather_rows_ring_kernel<C, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingMaxSmem);
    if (ge != cudaSuccess) return ge;
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int64_t blocks = ((int64_t)a.num_items + rc.warps - 1) / rc.warps;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  gather_rows_ring_kernel<C, R><<<(unsigned)blocks, rc.warps * 32, rc.smem, stream>>>(a, rc.cfg);
  return cudaGetLastError();
}

cudaError_t dispatch_ring(const GatherArgs& a, cudaStream_t stream) {
  const int nvec = (a.dim + 3) / 4;
  const RingChoice rc = choose_ring(nvec * 16);
  if (rc.smem > (size_t)kRingMaxSmem) return cudaErrorInvalidConfiguration;
  if (nvec <= 4) return launch_ring_one<1, 8>(a, rc, stream);
  if (nvec <= 8) return launch_ring_one<1, 4>(a, rc, stream);
  if (nvec <= 16) return launch_ring_one<1, 2>(a, rc, stream);
  switch ((nvec + 31) / 32) {
    case 1: return launch_ring_one<1, 1>(a, rc, stream);
    case 2: return launch_ring_one<2, 1>(a, rc, stream);
    case 3: return launch_ring_one<3, 1>(a, rc, stream);
    case 4: return launch_ring_one<4, 1>(a, rc, stream);
    case 5: return launch_ring_one<5, 1>(a, rc, stream);
    case 6: return launch_ring_one<6, 1>(a, rc, stream);
    default: return launch_ring_one<8, 1>(a, rc, stream);
  }
}

// ---- tile kernel launch -------------------------------------------------------------------
template <int L, int C, int U>
cudaError_t launch_tiles_one(const GatherArgs& a, const TileArgs& t, cudaStream_t stream) {
  const size_t smem = (size_t)kTileMaxStage * L * C * sizeof(float4);
  if (smem > 48 * 1024) {   // the opt-in to more than 48 KB of dynamic shared memory is per device
    static bool configured[64] = {false};
    int dev = 0;
    cudaError_t ge = cudaGetDevice(&dev);
    if (ge != cudaSuccess) return ge;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      ge = cudaFuncSetAttribute(gather_tiles_kernel<L, C, U, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (ge == cudaSuccess)
        ge = cudaFuncSetAttribute(gather_tiles_kernel<L, C, U, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (ge != cudaSuccess) return ge;
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
  }
  if (a.weight_gcn)
    gather_tiles_kernel<L, C, U, true><<<(unsigned)t.num_tiles, 256, smem, stream>>>(a, t);
  else
    gather_tiles_kernel<L, C, U, false><<<(unsigned)t.num_tiles, 256, smem, stream>>>(a, t);
  return cudaGetLastError();
}

constexpr int kRingMaxDim = 8 * 32 * 4;  // widest row one ring launch covers

}  // namespace

// Widest load vector every row start of every gathered buffer allows (the ragged last vector
// of a row is read whole, so the leading dimension must cover it).
static int pick_vec(const GatherArgs& a) {
  auto ok = [&](int vec) {
    const size_t bytes = (size_t)vec * 4;
    const int64_t need = round_up_to(a.dim, vec);
    if (!aligned_to(a.x, bytes) || (a.ldx % vec) || a.ldx < need) return false;
    if (a.partials && (!aligned_to(a.partials, bytes) || (a.ldp % vec) || a.ldp < need)) return false;
    if (a.slots && (!aligned_to(a.slots, bytes) || (a.lds % vec) || a.lds < need)) return false;
    return true;
  };
  if (ok(4)) return 4;
  if (ok(2)) return 2;
  return 1;
}

static bool out_allows(const GatherArgs& a, int vec) {
  return a.out == nullptr || (aligned_to(a.out, (size_t)vec * 4) && (a.ldo % vec) == 0);
}

enum { kKernelLanes = 0, kKernelRing = 1 };

// ROF_KERNEL = "ring" | "lanes" forces one of the gather kernels wherever the buffers
// allow it (experiments, tests); unset: the host policy in GatherArgs::kernel decides
static int kernel_override() {
  const char* e = std::getenv("ROF_KERNEL");
  if (e == nullptr) return -1;
  if (e[0] == 'r') return kKernelRing;
  if (e[0] == 'l') return kKernelLanes;
  return -1;
}

// The ring kernel needs 16-byte aligned rows and does not weight rows.
static int pick_kernel(const GatherArgs& a, int vec) {
  if (vec != 4) return kKernelLanes;
  const int ov = kernel_override();
  int k = ov >= 0 ? ov : a.kernel;
  if (k == kKernelRing && a.weight_gcn) k = kKernelLanes;
  return k;
}

cudaError_t launch_gather(const GatherArgs& a0, cudaStream_t stream, int* launches) {
  if (a0.num_items <= 0 || a0.dim <= 0) return cudaSuccess;
  const int vec = pick_vec(a0);
  const int kernel = pick_kernel(a0, vec);
  const int tile = kernel != kKernelLanes ? kRingMaxDim : 16 * 32 * vec;  // widest column tile one launch covers
  for (int off = 0; off < a0.dim; off += tile) {
    GatherArgs a = a0;
    a.dim = min(tile, a0.dim - off);
    a.x = a0.x + off;
    if (a0.partials) a.partials = a0.partials + off;
    if (a0.out) a.out = a0.out + off;
    if (a0.slots) a.slots = a0.slots + off;
    if (a0.ep.bias) a.ep.bias = a0.ep.bias + off;
    if (a0.ep.self_x) a.ep.self_x = a0.ep.self_x + off;
    if (a0.mirror) {
      a.mirror = a0.mirror + off;
      // the 1.0 "ready" flag sits after the last column: only the last tile writes it
      a.mirror_flag_col = (off + a.dim == a0.dim) ? a.dim : -1;
    }
    a.out_vec = out_allows(a, vec) ? 1 : 0;
    // with column tiles the arrival counters would be hit once per tile: leave the split rows
    // to split_reduce_kernel then
    if (a0.dim > tile) a.arrive = nullptr;
    cudaError_t e;
    if (kernel == kKernelRing) e = dispatch_ring(a, stream);
    else e = (vec == 4) ? dispatch_width<4>(a, stream) : (vec == 2) ? dispatch_width<2>(a, stream)
                                                                   : dispatch_width<1>(a, stream);
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
  }
  return cudaSuccess;
}

bool tiles_supported(const GatherArgs& a) {
  if (a.dim <= 0 || a.dim > kTileMaxFloats) return false;
  if (std::getenv("ROF_KERNEL") != nullptr) return false;   // a forced kernel (experiments, tests) bypasses the tiles
  return pick_vec(a) == 4;
}

cudaError_t launch_gather_tiles(const GatherArgs& a0, const TileArgs& t, cudaStream_t stream, int* launches) {
  if (t.num_tiles <= 0 || a0.dim <= 0) return cudaSuccess;
  GatherArgs a = a0;
  a.out_vec = out_allows(a, 4) ? 1 : 0;
  const int nvec = (a.dim + 3) / 4;
  const bool narrow = lane_shape_override() != 0;   // measured on the community graph: 11-18 % faster at every width from 36 to 128
  cudaError_t e;
  if (nvec <= 4) e = launch_tiles_one<4, 1, 4>(a, t, stream);
  else if (nvec <= 8) e = launch_tiles_one<8, 1, 8>(a, t, stream);
  else if (nvec <= 16) e = narrow ? launch_tiles_one<8, 2, 4>(a, t, stream) : launch_tiles_one<16, 1, 8>(a, t, stream);
  else if (nvec <= 32) e = narrow ? launch_tiles_one<16, 2, 4>(a, t, stream) : launch_tiles_one<32, 1, 8>(a, t, stream);
  else e = launch_tiles_one<32, 2, 4>(a, t, stream);
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

bool gather_fuses_reduce(const GatherArgs& a) {
  if (a.arrive == nullptr || a.dim <= 0) return false;
  const int vec = pick_vec(a);
  return a.dim <= (pick_kernel(a, vec) != kKernelLanes ? kRingMaxDim : 16 * 32 * vec);
}

cudaError_t launch_split_reduce(const ReduceArgs& a, cudaStream_t stream) {
  if (a.num_rows <= 0 || a.dim <= 0) return cudaSuccess;
  const int threads = 256;
  const int64_t blocks = ((int64_t)a.num_rows * 32 + threads - 1) / threads;
  split_reduce_kernel<<<(unsigned)blocks, threads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_scale_rows(const float* x, int64_t ldx, const float* degrees, float* out, int64_t ldo,
                              int num_rows, int dim, int pad_to, int op, cudaStream_t stream) {
  if (num_rows <= 0 || pad_to <= 0) return cudaSuccess;
  const int64_t want = ((int64_t)num_rows * 32 + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  scale_rows_kernel<<<blocks, 256, 0, stream>>>(x, ldx, degrees, out, ldo, num_rows, dim, pad_to, op);
  return cudaGetLastError();
}

cudaError_t launch_probe_read(const void* buf, int64_t bytes, int repeats, float* sink, cudaStream_t stream) {
  if (bytes < 16 || repeats <= 0) return cudaSuccess;
  probe_read_kernel<<<148 * 8, 256, 0, stream>>>(reinterpret_cast<const float4*>(buf), bytes / 16, repeats, sink);
  return cudaGetLastError();
}

}  // namespace rof
