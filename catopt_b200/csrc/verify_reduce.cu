// Verify reduction: per-segment max|ref-out|, max|ref| and NaN flags in one
// streaming pass over both tensors (the reference makes four eager passes,
// catopt_torch/report.py:128-140).
//
// Bandwidth kernel.  Algorithmic bytes per segment = 2 * numel * sizeof(elem);
// nothing is written except 16 bytes per segment.  A persistent grid of
// 148 x kCtasPerSm CTAs walks contiguous runs of 32 KiB tiles, each thread
// keeping 8 independent 16-byte loads per tensor in flight; a running maximum
// stays in registers while consecutive tiles belong to the same segment and is
// merged with one atomicMax per CTA per segment.  Maxima of non-negative
// floats order like their bit patterns, so the merge is exact and its order
// does not matter: the result is deterministic.
#include "common.cuh"

namespace cb2 {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 8;                              // 16-byte vectors per thread per tile
constexpr int kVecsPerTile = kThreads * kUnroll;        // 2048 vectors = 32 KiB per tensor
constexpr int kCtasPerSm = 8;

struct Acc {
  float max_abs = 0.f;
  float max_ref = 0.f;
  uint32_t nan_diff = 0;
  uint32_t nan_ref = 0;
};

template <int DTYPE>
__device__ __forceinline__ void accum_elem(float r, float o, Acc& acc) {
  float d = r - o;
  if (DTYPE == CB2_BF16) d = round_to_bf16(d);  // torch rounds the bf16 difference
  acc.nan_diff |= (d != d);
  acc.nan_ref |= (r != r);
  acc.max_abs = fmaxf(acc.max_abs, fabsf(d));   // fmaxf drops a NaN operand
  acc.max_ref = fmaxf(acc.max_ref, fabsf(r));
}

template <int DTYPE>
__device__ __forceinline__ void accum_vec(const uint4& r, const uint4& o, Acc& acc) {
  const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
  const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (DTYPE == CB2_BF16) {
      accum_elem<DTYPE>(bf16lo_to_f32(rw[i]), bf16lo_to_f32(ow[i]), acc);
      accum_elem<DTYPE>(bf16hi_to_f32(rw[i]), bf16hi_to_f32(ow[i]), acc);
    } else {
      accum_elem<DTYPE>(__uint_as_float(rw[i]), __uint_as_float(ow[i]), acc);
    }
  }
}

// CTA-wide merge of the running accumulators into result[seg].
__device__ void flush(Acc& acc, float* result, int64_t seg, float* s_red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    acc.max_abs = fmaxf(acc.max_abs, __shfl_xor_sync(0xffffffffu, acc.max_abs, off));
    acc.max_ref = fmaxf(acc.max_ref, __shfl_xor_sync(0xffffffffu, acc.max_ref, off));
    acc.nan_diff |= __shfl_xor_sync(0xffffffffu, acc.nan_diff, off);
    acc.nan_ref |= __shfl_xor_sync(0xffffffffu, acc.nan_ref, off);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // s_red may still be read by the previous flush
  if (lane == 0) {
    s_red[warp * 4 + 0] = acc.max_abs;
    s_red[warp * 4 + 1] = acc.max_ref;
    s_red[warp * 4 + 2] = acc.nan_diff ? 1.f : 0.f;
    s_red[warp * 4 + 3] = acc.nan_ref ? 1.f : 0.f;
  }
  __syncthreads();
  if (threadIdx.x < 4) {
    float m = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) m = fmaxf(m, s_red[w * 4 + threadIdx.x]);
    // All four fields are non-negative floats: unsigned bit order == value order.
    atomicMax(reinterpret_cast<unsigned int*>(result + seg * 4 + threadIdx.x),
              __float_as_uint(m));
  }
  acc = Acc{};
}

__global__ void verify_clear_kernel(float* result, int64_t n) {
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i < n) result[i] = 0.f;
}

// Vector path: every segment starts 16-byte aligned.
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
verify_reduce_kernel(const uint4* __restrict__ ref, const uint4* __restrict__ out,
                     int64_t vecs_per_seg, int64_t tiles_per_seg, int64_t total_tiles,
                     int64_t tiles_per_cta, float* __restrict__ result) {
  __shared__ float s_red[(kThreads / 32) * 4];
  const int64_t t0 = blockIdx.x * tiles_per_cta;
  const int64_t t1 = min(t0 + tiles_per_cta, total_tiles);
  if (t0 >= t1) return;
  Acc acc;
  int64_t cur_seg = t0 / tiles_per_seg;
  for (int64_t t = t0; t < t1; ++t) {
    const int64_t seg = t / tiles_per_seg;
    if (seg != cur_seg) {
      flush(acc, result, cur_seg, s_red);
      cur_seg = seg;
    }
    const int64_t v0 = (t - seg * tiles_per_seg) * kVecsPerTile;
    const int64_t base = seg * vecs_per_seg;
    uint4 r[kUnroll], o[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t v = v0 + u * kThreads + threadIdx.x;
      if (v < vecs_per_seg) {
        r[u] = __ldcs(ref + base + v);
        o[u] = __ldcs(out + base + v);
      } else {
        r[u] = make_uint4(0, 0, 0, 0);
        o[u] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) accum_vec<DTYPE>(r[u], o[u], acc);
  }
  flush(acc, result, cur_seg, s_red);
}

// Element path: arbitrary alignment and the sub-vector tail of a segment.
// elems [e0,e1) of every segment; one CTA row per segment (grid.y).
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
verify_reduce_elems_kernel(const void* __restrict__ ref, const void* __restrict__ out,
                           int64_t numel_per_seg, int64_t e0, float* __restrict__ result) {
  __shared__ float s_red[(kThreads / 32) * 4];
  const int64_t seg = blockIdx.y;
  Acc acc;
  for (int64_t e = e0 + blockIdx.x * int64_t(kThreads) + threadIdx.x; e < numel_per_seg;
       e += int64_t(gridDim.x) * kThreads) {
    const int64_t i = seg * numel_per_seg + e;
    float r, o;
    if (DTYPE == CB2_BF16) {
      r = __bfloat162float(static_cast<const __nv_bfloat16*>(ref)[i]);
      o = __bfloat162float(static_cast<const __nv_bfloat16*>(out)[i]);
    } else {
      r = static_cast<const float*>(ref)[i];
      o = static_cast<const float*>(out)[i];
    }
    accum_elem<DTYPE>(r, o, acc);
  }
  flush(acc, result, seg, s_red);
}

template <int DTYPE>
int launch(const void* ref, const void* out, int64_t numel, int64_t n_seg, float* result,
           cudaStream_t st) {
  const int64_t esz = DTYPE == CB2_BF16 ? 2 : 4;
  const int64_t per_vec = 16 / esz;
  const int64_t n_res = n_seg * 4;
  verify_clear_kernel<<<unsigned((n_res + 255) / 256), 256, 0, st>>>(result, n_res);
  CB2_LAUNCH_CHECK();
  const bool vec_ok = aligned16(ref) && aligned16(out) &&
                      (n_seg == 1 || (numel * esz) % 16 == 0);
  int64_t done = 0;  // elements per segment covered by the vector kernel
  if (vec_ok && numel >= per_vec) {
    const int64_t vecs = numel / per_vec;
    const int64_t tiles_per_seg = (vecs + kVecsPerTile - 1) / kVecsPerTile;
    const int64_t total = tiles_per_seg * n_seg;
    int64_t grid = int64_t(kNumSMs) * kCtasPerSm;
    if (grid > total) grid = total;
    const int64_t per_cta = (total + grid - 1) / grid;
    grid = (total + per_cta - 1) / per_cta;
    // With n_seg > 1 the segment stride in vectors equals vecs (no tail).
    verify_reduce_kernel<DTYPE><<<unsigned(grid), kThreads, 0, st>>>(
        static_cast<const uint4*>(ref), static_cast<const uint4*>(out), vecs, tiles_per_seg,
        total, per_cta, result);
    CB2_LAUNCH_CHECK();
    done = vecs * per_vec;
  }
  if (done < numel) {
    const int64_t rest = numel - done;
    int64_t gx = (rest + kThreads - 1) / kThreads;
    if (gx > 64) gx = 64;
    for (int64_t s0 = 0; s0 < n_seg; s0 += 65535) {
      const int64_t ns = (n_seg - s0 < 65535) ? (n_seg - s0) : 65535;
      const dim3 grid{unsigned(gx), unsigned(ns), 1u};
      verify_reduce_elems_kernel<DTYPE><<<grid, kThreads, 0, st>>>(
          static_cast<const char*>(ref) + s0 * numel * esz,
          static_cast<const char*>(out) + s0 * numel * esz, numel, done, result + s0 * 4);
      CB2_LAUNCH_CHECK();
    }
  }
  return CB2_OK;
}

}  // namespace
}  // namespace cb2

extern "C" int cb2_verify_reduce(const void* ref, const void* out, int64_t numel_per_seg,
                                 int64_t n_seg, int dtype, float* result, void* stream) {
  if (!ref || !out || !result) return CB2_NULL_PTR;
  if (numel_per_seg <= 0 || n_seg <= 0) return CB2_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_BF16) {
    if ((reinterpret_cast<uintptr_t>(ref) | reinterpret_cast<uintptr_t>(out)) & 1) return CB2_BAD_ALIGN;
    return cb2::launch<CB2_BF16>(ref, out, numel_per_seg, n_seg, result, st);
  }
  if (dtype == CB2_F32) {
    if ((reinterpret_cast<uintptr_t>(ref) | reinterpret_cast<uintptr_t>(out)) & 3) return CB2_BAD_ALIGN;
    return cb2::launch<CB2_F32>(ref, out, numel_per_seg, n_seg, result, st);
  }
  return CB2_UNSUPPORTED_DTYPE;
}
