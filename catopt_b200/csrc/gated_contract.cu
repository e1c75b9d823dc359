// Gated contraction  o = (s . g) @ v : C-ABI entry point, the dispatch between
// the tensor-core kernel (gated_contract_tc.cu: bf16, K and dv multiples of 8,
// dv <= 128) and a general fp32-FMA kernel for everything else (fp32 tensors,
// odd sizes, wide values).  Semantics: `_om_decayed_torch`,
// catopt_carriers/om.py:1053-1057 — the elementwise product is rounded to the
// tensor dtype, the contraction accumulates in fp32, the result is rounded once.
#include "common.cuh"

namespace cb2 {

bool gated_contract_tc_supported(long long nb, int T, int K, int dv, int dtype, const void* s,
                                 const void* g, const void* v, const void* o);
int gated_contract_tc_run(const void* s, const void* g, const void* v, void* o, long long nb, long long ng,
                          int T, int K, int dv, int g_div, int g_mod, int* dev_status, cudaStream_t st);

namespace {

template <typename T>
__device__ __forceinline__ float ld_elem(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld_elem<float>(const float* p, size_t i) { return __ldg(p + i); }
template <>
__device__ __forceinline__ float ld_elem<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(p[i]);
}
template <typename T>
__device__ __forceinline__ float round_elem(float x);
template <>
__device__ __forceinline__ float round_elem<float>(float x) { return x; }
template <>
__device__ __forceinline__ float round_elem<__nv_bfloat16>(float x) { return round_to_bf16(x); }
template <typename T>
__device__ __forceinline__ void st_elem(T* p, size_t i, float x);
template <>
__device__ __forceinline__ void st_elem<float>(float* p, size_t i, float x) { p[i] = x; }
template <>
__device__ __forceinline__ void st_elem<__nv_bfloat16>(__nv_bfloat16* p, size_t i, float x) {
  p[i] = __float2bfloat16_rn(x);
}

constexpr int kFT = 64;   // output tile: 64 rows x 64 value columns
constexpr int kFK = 16;   // keys per slab

// CTA = one 64 x 64 output tile of one batch; 256 threads, 4 x 4 outputs each.
template <typename T>
__global__ void __launch_bounds__(256)
gated_contract_ffma_kernel(const T* __restrict__ s, const T* __restrict__ g, const T* __restrict__ v,
                           T* __restrict__ o, int Tq, int K, int dv, int row_tiles, int g_div, int g_mod) {
  __shared__ float sp[kFK][kFT + 1];   // P slab, transposed: [key][row]
  __shared__ float sv[kFK][kFT];       // V slab: [key][column]
  const int b = blockIdx.x / row_tiles;
  const int row0 = (blockIdx.x % row_tiles) * kFT;
  const int col0 = blockIdx.y * kFT;
  const int gb = (b / g_div) % g_mod;
  const T* sb = s + size_t(b) * Tq * K;
  const T* gp = g + size_t(gb) * Tq * K;
  const T* vb = v + size_t(b) * K * dv;
  const int tid = threadIdx.x;
  const int tr = (tid >> 4) * 4, tc = (tid & 15) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += kFK) {
    // P slab: thread loads (row = tid / 4 .. , 4 keys)
    {
      const int r = tid >> 2, kk = (tid & 3) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = row0 + r, key = k0 + kk + e;
        float p = 0.f;
        if (row < Tq && key < K) {
          const size_t i = size_t(row) * K + key;
          p = round_elem<T>(ld_elem<T>(sb, i) * ld_elem<T>(gp, i));
        }
        sp[kk + e][r] = p;
      }
    }
    {
      const int kk = tid >> 4, c = (tid & 15) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + kk, col = col0 + c + e;
        sv[kk][c + e] = (key < K && col < dv) ? ld_elem<T>(vb, size_t(key) * dv + col) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kFK; ++kk) {
      float pr[4], vc[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) { pr[e] = sp[kk][tr + e]; vc[e] = sv[kk][tc + e]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(pr[i], vc[j], acc[i][j]);
    }
    __syncthreads();
  }
  T* ob = o + size_t(b) * Tq * dv;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = row0 + tr + i, col = col0 + tc + j;
      if (row < Tq && col < dv) st_elem<T>(ob, size_t(row) * dv + col, acc[i][j]);
    }
}

template <typename T>
int run_ffma(const void* s, const void* g, const void* v, void* o, long long nb, int Tq, int K, int dv,
             int g_div, int g_mod, cudaStream_t st) {
  const int row_tiles = (Tq + kFT - 1) / kFT;
  const long long gx = nb * row_tiles;
  const int gy = (dv + kFT - 1) / kFT;
  if (gx >= (1ll << 31) || gy > 65535) return CB2_BAD_SHAPE;
  gated_contract_ffma_kernel<T><<<dim3(unsigned(gx), unsigned(gy)), 256, 0, st>>>(
      static_cast<const T*>(s), static_cast<const T*>(g), static_cast<const T*>(v), static_cast<T*>(o), Tq, K,
      dv, row_tiles, g_div, g_mod);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace
}  // namespace cb2

extern "C" int cb2_gated_contract_on_tensor_cores(long long nb, int T, int K, int dv, int dtype) {
  return cb2::gated_contract_tc_supported(nb, T, K, dv, dtype, nullptr, nullptr, nullptr, nullptr) ? 1 : 0;
}

extern "C" int cb2_gated_contract_fwd(const void* s, const void* g, const void* v, void* o, long long nb,
                                      long long ng, int T, int K, int dv, int g_div, int g_mod, int dtype,
                                      int* dev_status, void* stream) {
  if (!s || !g || !v || !o) return CB2_NULL_PTR;
  if (nb <= 0 || ng <= 0 || T <= 0 || K <= 0 || dv <= 0 || g_div <= 0 || g_mod <= 0 || g_mod > ng)
    return CB2_BAD_SHAPE;
  if (dtype != CB2_F32 && dtype != CB2_BF16) return CB2_UNSUPPORTED_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cb2::gated_contract_tc_supported(nb, T, K, dv, dtype, s, g, v, o))
    return cb2::gated_contract_tc_run(s, g, v, o, nb, ng, T, K, dv, g_div, g_mod, dev_status, st);
  if (dtype == CB2_F32) return cb2::run_ffma<float>(s, g, v, o, nb, T, K, dv, g_div, g_mod, st);
  return cb2::run_ffma<__nv_bfloat16>(s, g, v, o, nb, T, K, dv, g_div, g_mod, st);
}
