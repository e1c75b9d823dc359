// Start states of sequence segments for the diagonal scan
//     h_t[n] = a_t[n] h_(t-1)[n] + b[n] x_t,
// so that a scan with few (batch, channel-block) units can run its segments side by side.
// One step is the reference's `applyd(aff_diag(a_t, b*x_t), h)` (catopt_torch/
// torch_bridge.py:1895-1900) and steps compose by `affd_compose` (:1896-1899), so the
// state a segment starts from follows from the composed maps of the segments before it:
//
//   kernel 1: (A_s, U_s) = composed map of a piece of a segment (up to 8 pieces per
//             segment): A_s = prod a_t, U_s = the state the piece ends in when started
//             from zero; every thread owns four state
//             elements of one channel and walks the segment with eight steps of loads in
//             flight (one pass over a and x);
//   kernel 2: S_0 = h0 (or 0), S_s = A_(s-1) S_(s-1) + U_(s-1), fp32.
//
// The caller then runs cb2_diag_scan_fwd on the [B*n_seg, T/n_seg, ...] view of the same
// tensors with these start states: `a` and x are read twice, which pays while the
// one-pass form keeps fewer than half the SMs busy.
#include "common.cuh"

namespace cb2 {
namespace {

constexpr int kSegThreads = 128;
constexpr int kSegUnroll = 8;

template <int DTYPE>
struct Ld4;
template <>
struct Ld4<CB2_F32> {
  __device__ static void ld(const void* p, size_t i, float (&v)[4]) {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i));
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  __device__ static float ld1(const void* p, size_t i) { return __ldg(static_cast<const float*>(p) + i); }
};
template <>
struct Ld4<CB2_BF16> {
  __device__ static void ld(const void* p, size_t i, float (&v)[4]) {
    const uint2 x = __ldcs(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + i));
    v[0] = bf16lo_to_f32(x.x); v[1] = bf16hi_to_f32(x.x);
    v[2] = bf16lo_to_f32(x.y); v[3] = bf16hi_to_f32(x.y);
  }
  __device__ static float ld1(const void* p, size_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
};

// grid: (state elements / 4 / 128, n_seg, B)
template <int DTYPE>
__global__ void __launch_bounds__(kSegThreads)
scan_seg_maps_kernel(const void* __restrict__ a, const void* __restrict__ x, const void* __restrict__ bmat,
                     int T, int D, int N, int seg_len, float* __restrict__ seg_a, float* __restrict__ seg_u) {
  using L = Ld4<DTYPE>;
  const int e0 = (blockIdx.x * kSegThreads + threadIdx.x) * 4;     // first of four state elements (same channel)
  const int DN = D * N;
  if (e0 >= DN) return;
  const int d = e0 / N;
  const int seg = blockIdx.y, n_seg = gridDim.y, bb = blockIdx.z;
  const int t0 = seg * seg_len;
  const int t1 = min(T, t0 + seg_len);
  float bw[4];
  L::ld(bmat, size_t(e0), bw);
  float A[4] = {1.f, 1.f, 1.f, 1.f}, U[4] = {0.f, 0.f, 0.f, 0.f};
  const size_t a_base = size_t(bb) * T * DN + size_t(e0);
  const size_t x_base = size_t(bb) * T * D + size_t(d);
  int t = t0;
  for (; t + kSegUnroll <= t1; t += kSegUnroll) {
    float av[kSegUnroll][4], xv[kSegUnroll];
#pragma unroll
    for (int u = 0; u < kSegUnroll; ++u) {
      L::ld(a, a_base + size_t(t + u) * DN, av[u]);
      xv[u] = L::ld1(x, x_base + size_t(t + u) * D);
    }
#pragma unroll
    for (int u = 0; u < kSegUnroll; ++u)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        U[j] = fmaf(av[u][j], U[j], bw[j] * xv[u]);
        A[j] *= av[u][j];
      }
  }
  for (; t < t1; ++t) {
    float av[4];
    L::ld(a, a_base + size_t(t) * DN, av);
    const float xv = L::ld1(x, x_base + size_t(t) * D);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      U[j] = fmaf(av[j], U[j], bw[j] * xv);
      A[j] *= av[j];
    }
  }
  const size_t o = (size_t(bb) * n_seg + seg) * DN + e0;
  *reinterpret_cast<float4*>(seg_a + o) = make_float4(A[0], A[1], A[2], A[3]);
  *reinterpret_cast<float4*>(seg_u + o) = make_float4(U[0], U[1], U[2], U[3]);
}

// starts[b][s][e]: S_0 = h0 (or 0), S_s = A_(s-1) S_(s-1) + U_(s-1).  The maps come in
// pieces finer than the segments (`fine` pieces per segment, so that kernel 1 has enough
// threads to stream at full rate); a start state is written at every segment boundary.
__global__ void __launch_bounds__(256)
scan_seg_starts_kernel(const float* __restrict__ seg_a, const float* __restrict__ seg_u,
                       const float* __restrict__ h0, int DN, int n_seg, int fine, float* __restrict__ starts) {
  const int e = blockIdx.x * 256 + threadIdx.x;
  if (e >= DN) return;
  const int bb = blockIdx.y;
  float s = h0 ? h0[size_t(bb) * DN + e] : 0.f;
  for (int sg = 0; sg < n_seg; ++sg) {
    starts[(size_t(bb) * n_seg + sg) * DN + e] = s;
    for (int f = 0; f < fine; ++f) {
      const size_t o = (size_t(bb) * n_seg * fine + size_t(sg) * fine + f) * DN + e;
      s = fmaf(seg_a[o], s, seg_u[o]);
    }
  }
}

// pieces per segment for kernel 1: up to 8, at least 64 steps each
int fine_pieces(int seg_len) {
  for (int f = 8; f > 1; f /= 2)
    if (seg_len % f == 0 && seg_len / f >= 64) return f;
  return 1;
}

template <int DTYPE>
int run_seg(const void* a, const void* x, const void* b, const float* h0, int B, int T, int D, int N, int n_seg,
            float* starts, float* scratch, cudaStream_t st) {
  const int DN = D * N;
  const int fine = fine_pieces(T / n_seg);
  const int n_fine = n_seg * fine;
  if (n_fine > 65535) return CB2_BAD_SHAPE;
  const int piece_len = T / n_fine;
  float* seg_a = scratch;
  float* seg_u = scratch + size_t(B) * n_fine * DN;
  const dim3 grid(unsigned((DN / 4 + kSegThreads - 1) / kSegThreads), unsigned(n_fine), unsigned(B));
  scan_seg_maps_kernel<DTYPE><<<grid, kSegThreads, 0, st>>>(a, x, b, T, D, N, piece_len, seg_a, seg_u);
  CB2_LAUNCH_CHECK();
  scan_seg_starts_kernel<<<dim3(unsigned((DN + 255) / 256), unsigned(B)), 256, 0, st>>>(seg_a, seg_u, h0, DN, n_seg,
                                                                                       fine, starts);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace
}  // namespace cb2

extern "C" size_t cb2_diag_scan_seg_scratch_bytes(int B, int D, int N, int n_seg) {
  if (B <= 0 || D <= 0 || N <= 0 || n_seg <= 0) return 0;
  return size_t(2) * B * n_seg * 8 * D * N * sizeof(float);   // up to 8 pieces per segment
}

extern "C" int cb2_diag_scan_seg_starts(const void* a, const void* x, const void* b, const float* h0,
                                        float* starts, int B, int T, int D, int N, int n_seg, int dtype,
                                        void* scratch, size_t scratch_bytes, void* stream) {
  if (!a || !x || !b || !starts) return CB2_NULL_PTR;
  if (B <= 0 || T <= 0 || D <= 0 || N <= 0 || n_seg <= 0 || T % n_seg != 0 || N % 4 != 0 || B > 65535 ||
      n_seg > 65535)
    return CB2_BAD_SHAPE;
  if (!cb2::aligned16(a) || !cb2::aligned16(b) || !cb2::aligned16(starts)) return CB2_BAD_ALIGN;
  if (!scratch || !cb2::aligned16(scratch) || scratch_bytes < cb2_diag_scan_seg_scratch_bytes(B, D, N, n_seg))
    return CB2_SCRATCH_TOO_SMALL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_F32)
    return cb2::run_seg<CB2_F32>(a, x, b, h0, B, T, D, N, n_seg, starts, static_cast<float*>(scratch), st);
  if (dtype == CB2_BF16)
    return cb2::run_seg<CB2_BF16>(a, x, b, h0, B, T, D, N, n_seg, starts, static_cast<float*>(scratch), st);
  return CB2_UNSUPPORTED_DTYPE;
}
