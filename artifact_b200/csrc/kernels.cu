// Gather kernels for sm_100a.
//
// One kernel template does all the summing: a *lane group* of L threads (L = 4..32, a
// power of two chosen from the feature width) owns one work item — a destination row, one
// segment of a long destination row, or one reuse group — and walks the item's entries.
// The group fetches L column entries with one coalesced load, broadcasts them with
// shuffles, and issues U independent 128-bit (or 64/32-bit when the width forces it) row
// loads per lane before accumulating, so that each warp keeps U*C*16 B per lane in flight.
// Accumulators live in registers; every output row is stored exactly once, so there are no
// atomics and no zero-fill pass (upstream: atomicAdd_F per element per part and a
// torch::zeros per call, reuse_conv_kernel.cu:16-21, 282, 303).
//
// The kernel is bound by instruction issue before it is bound by L2 or HBM (hub rows are
// re-read from L2), so the inner loop is kept to one shuffle, one 64-bit multiply-add and
// the loads and adds per entry: an item's entries are ordered [partial rows | feature rows]
// so each range has a fixed base pointer, the unweighted modes (sum, mean, partial rows) do
// no multiply at all, and full batches run without per-entry predicates.
//
// Arithmetic: sum/mean add the gathered values (rounded to nearest); GCN adds
// rsqrt_rn(degrees[src]) * x with one fused multiply-add per term — a single rounding where
// upstream has two (__fmul_rn then add, reuse_conv_kernel.cu:254, 270); the order of the adds
// differs from upstream's (arbitrary atomic order) in any case.
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

// out = act(r + self_scale * self_x[row][col..] + bias[col..]) for VEC consecutive columns.
// The pointers need no alignment: the epilogue reads scalars.
template <int VEC>
__device__ __forceinline__ void apply_epilogue(float (&r)[VEC], const Epilogue& ep, int row, int col) {
  if (ep.self_x != nullptr) {
    const float* sp = ep.self_x + (int64_t)row * ep.ld_self + col;
#pragma unroll
    for (int t = 0; t < VEC; ++t) r[t] = __fmaf_rn(ep.self_scale, __ldg(sp + t), r[t]);
  }
  if (ep.bias != nullptr) {
#pragma unroll
    for (int t = 0; t < VEC; ++t) r[t] = __fadd_rn(r[t], __ldg(ep.bias + col + t));
  }
  if (ep.relu) {
#pragma unroll
    for (int t = 0; t < VEC; ++t) r[t] = fmaxf(r[t], 0.0f);
  }
}

// acc += sum over col[begin, end) of (WEIGHTED ? rsqrt(degrees[c]) : 1) * row(c), where
// row(c) starts at base_lane + (c - c_offset) * ld (base_lane already includes this lane's
// column offset).  `active[k]` says whether this lane's k-th vector lies inside the row.
template <int VEC, int L, int C, int U, bool WEIGHTED>
__device__ __forceinline__ void accumulate_range(float (&acc)[C][VEC], const int32_t* __restrict__ col, int begin,
                                                 int end, const float* base_lane, int64_t ld, int c_offset,
                                                 const float* __restrict__ degrees, int lane, unsigned gmask,
                                                 const bool (&active)[C]) {
  for (int e = begin; e < end; e += L) {
    const int mine = e + lane;
    int c = 0;
    float w = 1.0f;
    if (mine < end) {
      c = __ldg(col + mine);
      if constexpr (WEIGHTED) w = __frsqrt_rn(__ldg(degrees + c));
      c -= c_offset;
    }
    const int cnt = min(L, end - e);
    int j = 0;
    for (; j + U <= cnt; j += U) {  // full batches: no per-entry predicate
      float v[U][C][VEC];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int cj = __shfl_sync(gmask, c, j + u, L);
        const float* rp = base_lane + (int64_t)cj * ld;
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
      for (int u = 0; u < U; ++u) {
        float wj = 1.0f;
        if constexpr (WEIGHTED) wj = __shfl_sync(gmask, w, j + u, L);
#pragma unroll
        for (int k = 0; k < C; ++k)
#pragma unroll
          for (int t = 0; t < VEC; ++t) {
            if constexpr (WEIGHTED) acc[k][t] = __fmaf_rn(wj, v[u][k][t], acc[k][t]);
            else acc[k][t] = __fadd_rn(acc[k][t], v[u][k][t]);
          }
      }
    }
    if (j < cnt) {  // the last, partial batch of the range: same shape, predicated per entry
      float v[U][C][VEC];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int cj = __shfl_sync(gmask, c, j + u, L);
        const bool ok = (j + u) < cnt;
        const float* rp = base_lane + (int64_t)cj * ld;
#pragma unroll
        for (int k = 0; k < C; ++k) {
          if (ok && active[k]) {
            load_row_vec<VEC>(v[u][k], rp + k * (L * VEC));
          } else {
#pragma unroll
            for (int t = 0; t < VEC; ++t) v[u][k][t] = 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float wj = 1.0f;
        if constexpr (WEIGHTED) wj = __shfl_sync(gmask, w, j + u, L);
        if ((j + u) < cnt) {
#pragma unroll
          for (int k = 0; k < C; ++k)
#pragma unroll
            for (int t = 0; t < VEC; ++t) {
              if constexpr (WEIGHTED) acc[k][t] = __fmaf_rn(wj, v[u][k][t], acc[k][t]);
              else acc[k][t] = __fadd_rn(acc[k][t], v[u][k][t]);
            }
        }
      }
    }
  }
}

// VEC floats per load, L lanes per item, C vectors per lane (L*C*VEC >= dim), U rows in flight;
// WEIGHTED: multiply each feature row by rsqrt(degrees[col]) (GCN).
template <int VEC, int L, int C, int U, bool WEIGHTED>
__global__ void __launch_bounds__(256, (C <= 2 ? 4 : 1)) gather_rows_kernel(const GatherArgs a) {
  static_assert(U <= L && (L % U) == 0, "a batch of L entries is a whole number of unrolled steps");
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int item_id = (int)(gtid / L);
  if (item_id >= a.num_items) return;  // whole lane groups leave together
  const int lane = threadIdx.x & (L - 1);
  const unsigned gmask = (L == 32) ? 0xffffffffu : (((1u << L) - 1u) << ((threadIdx.x & 31) & ~(L - 1)));

  const int4 raw = __ldg(reinterpret_cast<const int4*>(a.items) + item_id);
  const int begin = raw.x, end = raw.y, dst = raw.z, mid = raw.w;  // [begin,mid) partial rows, [mid,end) feature rows
  const int nvec = a.dim / VEC;

  bool active[C];
  float acc[C][VEC];
#pragma unroll
  for (int k = 0; k < C; ++k) {
    active[k] = (lane + k * L) < nvec;
#pragma unroll
    for (int t = 0; t < VEC; ++t) acc[k][t] = 0.0f;
  }

  if (mid > begin)
    accumulate_range<VEC, L, C, U, false>(acc, a.col, begin, mid, a.partials + lane * VEC, a.ldp, a.num_nodes,
                                          nullptr, lane, gmask, active);
  if (end > mid)
    accumulate_range<VEC, L, C, U, WEIGHTED>(acc, a.col, mid, end, a.x + lane * VEC, a.ldx, 0, a.degrees, lane,
                                             gmask, active);

  float scale = 1.0f;
  float* op;
  if (dst >= 0) {
    if (begin == end) {
      // a row without entries is exactly zero whatever its degree says (upstream never
      // touches it after the zero-fill); 0 * rsqrt(0) would be NaN
      scale = 0.0f;
    } else if (a.scale_mode == 1) {
      scale = __frsqrt_rn(__ldg(a.degrees + dst));
    } else if (a.scale_mode == 2) {
      const float d = __ldg(a.degrees + dst);
      scale = (d == 0.0f) ? 0.0f : __frcp_rn(d);
    }
    op = a.out + (int64_t)(dst - a.row_begin) * a.ldo;
  } else {
    op = a.slots + (int64_t)(-dst - 1) * a.lds;
  }
#pragma unroll
  for (int k = 0; k < C; ++k) {
    if (active[k]) {
      const int iv = lane + k * L;
      float r[VEC];
#pragma unroll
      for (int t = 0; t < VEC; ++t) r[t] = __fmul_rn(acc[k][t], scale);
      if (a.accumulate && dst >= 0) {  // a later stage of a staged pass adds to the row
        const float* prev = op + (int64_t)iv * VEC;
#pragma unroll
        for (int t = 0; t < VEC; ++t) r[t] = __fadd_rn(prev[t], r[t]);
      }
      if (dst >= 0) apply_epilogue<VEC>(r, a.ep, dst, iv * VEC);
      store_row_vec<VEC>(op + (int64_t)iv * VEC, r);
      if (a.mirror != nullptr && dst >= 0) {
        float* mp = a.mirror + (int64_t)dst * a.ldm + (int64_t)iv * VEC;
#pragma unroll
        for (int t = 0; t < VEC; ++t) mp[t] = r[t];
      }
    }
  }
  if (a.mirror != nullptr && a.mirror_flag_col >= 0 && dst >= 0 && lane == 0)
    a.mirror[(int64_t)dst * a.ldm + a.mirror_flag_col] = 1.0f;
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
    apply_epilogue<1>(r, a.ep, row, d);
    op[d] = r[0];
  }
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

template <int VEC>
cudaError_t dispatch_width(const GatherArgs& a, cudaStream_t stream) {
  const int nvec = a.dim / VEC;
  if (nvec <= 4) return launch_one<VEC, 4, 1, 4>(a, stream);
  if (nvec <= 8) return launch_one<VEC, 8, 1, 8>(a, stream);
  if (nvec <= 16) return launch_one<VEC, 16, 1, 8>(a, stream);
  const int c = (nvec + 31) / 32;
  switch (c) {
    case 1: return launch_one<VEC, 32, 1, 8>(a, stream);
    case 2: return launch_one<VEC, 32, 2, 4>(a, stream);
    case 3: return launch_one<VEC, 32, 3, 2>(a, stream);
    case 4: return launch_one<VEC, 32, 4, 2>(a, stream);
    case 5: return launch_one<VEC, 32, 5, 2>(a, stream);
    case 6: return launch_one<VEC, 32, 6, 2>(a, stream);
    case 7: case 8: return launch_one<VEC, 32, 8, 1>(a, stream);
    case 9: case 10: return launch_one<VEC, 32, 10, 1>(a, stream);
    case 11: case 12: return launch_one<VEC, 32, 12, 1>(a, stream);
    default: return launch_one<VEC, 32, 16, 1>(a, stream);
  }
}

inline bool aligned_to(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

}  // namespace

// Widest vector every row start of every buffer touched allows.
static int pick_vec(const GatherArgs& a) {
  auto ok = [&](int vec) {
    const size_t bytes = (size_t)vec * 4;
    if (a.dim % vec) return false;
    if (!aligned_to(a.x, bytes) || (a.ldx % vec)) return false;
    if (a.partials && (!aligned_to(a.partials, bytes) || (a.ldp % vec))) return false;
    if (a.out && (!aligned_to(a.out, bytes) || (a.ldo % vec))) return false;
    if (a.slots && (!aligned_to(a.slots, bytes) || (a.lds % vec))) return false;
    return true;
  };
  if (ok(4)) return 4;
  if (ok(2)) return 2;
  return 1;
}

cudaError_t launch_gather(const GatherArgs& a0, cudaStream_t stream) {
  if (a0.num_items <= 0 || a0.dim <= 0) return cudaSuccess;
  const int vec = pick_vec(a0);
  const int tile = 16 * 32 * vec;  // widest column tile one launch covers (C=16, L=32)
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
    const cudaError_t e = (vec == 4)   ? dispatch_width<4>(a, stream)
                          : (vec == 2) ? dispatch_width<2>(a, stream)
                                       : dispatch_width<1>(a, stream);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_split_reduce(const ReduceArgs& a, cudaStream_t stream) {
  if (a.num_rows <= 0 || a.dim <= 0) return cudaSuccess;
  const int threads = 256;
  const int64_t blocks = ((int64_t)a.num_rows * 32 + threads - 1) / threads;
  split_reduce_kernel<<<(unsigned)blocks, threads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace rof
