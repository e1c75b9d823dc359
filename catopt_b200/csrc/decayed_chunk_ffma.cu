// Chunked decayed attention on the fp32 FMA pipes: the path used for fp32
// tensors (rel-err budget 1e-5, out of reach of a TF32 tensor-core pass) and
// for shapes the tensor-core kernel does not cover.
//
//   o[t] = sum_{s<=t} g^(t-s) (q_t . k_s) v_s / scale          per (batch, head)
//
// is evaluated chunk-wise with a carried state instead of the reference's
// all-pairs cross products (decayed_lower.py:671-700):
//   1. P_i  = (Q_i K_i^T) . tril(g^(r-c))                 -> scratch (fp32)
//      KV_i = (K_i . g^(C-1-r))^T V_i                     -> scratch (fp32)
//   2. S_0 = 0, S_{i+1} = g^C S_i + KV_i                  (in place: KV_i <- S_i)
//   3. O_i  = ( P_i V_i + diag(g^(r+1)) Q_i S_i ) / scale -> o
// Steps 1 and 3 are independent over (b, h, chunk) and fill the GPU even when
// B*H is small; step 2 is an elementwise scan over the chunk axis.  Powers of
// gamma are tabulated per CTA in shared memory (powf, fp32).  Three launches:
// one kernel does every P and KV tile of step 1, one the scan, one step 3.
//
// scratch layout (floats): [B*H*K][C][C] P | [B*H*K][dk][dv] KV/S
#include "common.cuh"

namespace cb2 {
namespace {

constexpr int kTile = 64;
constexpr int kSlice = 16;
constexpr int kThreads = 256;

template <int DTYPE>
__device__ __forceinline__ float ld_elem(const void* p, size_t i) {
  if (DTYPE == CB2_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return static_cast<const float*>(p)[i];
}
template <int DTYPE>
__device__ __forceinline__ void st_elem(void* p, size_t i, float v) {
  if (DTYPE == CB2_BF16)
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else
    static_cast<float*>(p)[i] = v;
}

constexpr int kMaxChunk = 1024;   // size of the per-CTA power table

// s_pw[k] = g^k for k in [0, C]; ends with a CTA barrier.
__device__ __forceinline__ void fill_pow_table(float* s_pw, float g, int C) {
  for (int k = threadIdx.x; k <= C; k += blockDim.x) s_pw[k] = powf(g, float(k));
  __syncthreads();
}

// acc += A_tile . B_tile over k in [0,kdim), 64x64 output tile at (m0,n0).
// fa(m,k) / fb(k,n) return the operand element (0 outside the matrix).
// A_KCONTIG / B_NCONTIG pick the thread->element mapping that makes the global
// reads of the operand contiguous.
template <bool A_KCONTIG, bool B_NCONTIG, class FA, class FB>
__device__ __forceinline__ void tile_gemm(float (&acc)[4][4], int kdim, FA fa, FB fb,
                                          float (*As)[kTile + 4], float (*Bs)[kTile + 4]) {
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  for (int k0 = 0; k0 < kdim; k0 += kSlice) {
    if (A_KCONTIG) {
      const int r = tid / 4, kq = (tid % 4) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) As[kq + j][r] = fa(r, k0 + kq + j);
    } else {
      const int kk = tid / 16, mq = (tid % 16) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) As[kk][mq + j] = fa(mq + j, k0 + kk);
    }
    if (B_NCONTIG) {
      const int kk = tid / 16, nq = (tid % 16) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) Bs[kk][nq + j] = fb(k0 + kk, nq + j);
    } else {
      const int r = tid / 4, kq = (tid % 4) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) Bs[kq + j][r] = fb(k0 + kq + j, r);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSlice; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a4[4] = {av.x, av.y, av.z, av.w};
      const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }
}

// Step 1, one launch: blockIdx.y < ct*ct is a 64x64 tile of
//   P[z] = (Q_i K_i^T) . tril(g^(r-c))
// and the remaining blockIdx.y values are 64x64 tiles of
//   KV[z] = (K_i . g^(C-1-r))^T V_i.
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
chunk_local_kernel(const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                   const float* __restrict__ gamma, float* __restrict__ P, float* __restrict__ KV, int H,
                   int T, int dk, int dv, int C, int ct, int vt) {
  __shared__ __align__(16) float As[kSlice][kTile + 4];
  __shared__ __align__(16) float Bs[kSlice][kTile + 4];
  __shared__ float s_pw[kMaxChunk + 1];
  const int nchunk = T / C;
  const int z = blockIdx.x, bh = z / nchunk, i = z % nchunk, h = bh % H;
  fill_pow_table(s_pw, gamma[h], C);
  const float* pw = s_pw;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  const size_t kbase = (size_t(bh) * T + size_t(i) * C) * dk;
  const size_t vbase = (size_t(bh) * T + size_t(i) * C) * dv;
  if (int(blockIdx.y) < ct * ct) {
    const int m0 = (blockIdx.y / ct) * kTile, n0 = (blockIdx.y % ct) * kTile;
    float* out = P + size_t(z) * C * C;
    if (n0 <= m0 + kTile - 1) {  // tiles strictly above the diagonal are all zero
      auto fa = [&](int m, int kk) {
        return (m0 + m < C && kk < dk) ? ld_elem<DTYPE>(q, kbase + size_t(m0 + m) * dk + kk) : 0.f;
      };
      auto fb = [&](int kk, int n) {
        return (n0 + n < C && kk < dk) ? ld_elem<DTYPE>(k, kbase + size_t(n0 + n) * dk + kk) : 0.f;
      };
      tile_gemm<true, false>(acc, dk, fa, fb, As, Bs);
    }
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int r = m0 + ty * 4 + ii;
      if (r >= C) continue;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int c = n0 + tx * 4 + jj;
        if (c < C) out[size_t(r) * C + c] = (c <= r) ? acc[ii][jj] * pw[r - c] : 0.f;
      }
    }
    return;
  }
  const int t = blockIdx.y - ct * ct;
  const int m0 = (t / vt) * kTile, n0 = (t % vt) * kTile;
  auto fa = [&](int m, int r) {  // A[m=e][k=r] = K[r][e] * g^(C-1-r)
    return (m0 + m < dk && r < C) ? ld_elem<DTYPE>(k, kbase + size_t(r) * dk + m0 + m) * pw[C - 1 - r]
                                  : 0.f;
  };
  auto fb = [&](int r, int n) {
    return (n0 + n < dv && r < C) ? ld_elem<DTYPE>(v, vbase + size_t(r) * dv + n0 + n) : 0.f;
  };
  tile_gemm<false, true>(acc, C, fa, fb, As, Bs);
  float* out = KV + size_t(z) * dk * dv;
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    const int e = m0 + ty * 4 + ii;
    if (e >= dk) continue;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int f = n0 + tx * 4 + jj;
      if (f < dv) out[size_t(e) * dv + f] = acc[ii][jj];
    }
  }
}

// Step 2: exclusive decayed scan over chunks, in place (KV_i <- S_i).  Eight
// chunks are loaded before the dependent FMA chain runs, so the loads overlap.
__global__ void state_scan_kernel(float* __restrict__ KV, const float* __restrict__ gamma, int H,
                                  int nchunk, int C, size_t per_chunk, size_t total_bh) {
  const size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (idx >= total_bh * per_chunk) return;
  const size_t bh = idx / per_chunk, e = idx % per_chunk;
  const float gC = powf(gamma[bh % H], float(C));
  float* p = KV + bh * nchunk * per_chunk + e;
  float state = 0.f;
  for (int i0 = 0; i0 < nchunk; i0 += 8) {
    float kv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) kv[j] = (i0 + j < nchunk) ? p[size_t(i0 + j) * per_chunk] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (i0 + j < nchunk) p[size_t(i0 + j) * per_chunk] = state;
      state = fmaf(gC, state, kv[j]);
    }
  }
}

// Step 3: O_i = (P_i V_i + diag(g^(r+1)) Q_i S_i) / scale.  grid (batch, C/64, dv/64)
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
output_kernel(const void* __restrict__ q, const void* __restrict__ v, const float* __restrict__ gamma,
              const float* __restrict__ P, const float* __restrict__ S, void* __restrict__ o, int H,
              int T, int dk, int dv, int C, float scale) {
  __shared__ __align__(16) float As[kSlice][kTile + 4];
  __shared__ __align__(16) float Bs[kSlice][kTile + 4];
  __shared__ float s_pw[kMaxChunk + 1];
  const int nchunk = T / C;
  const int z = blockIdx.x, bh = z / nchunk, i = z % nchunk, h = bh % H;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.z * kTile;
  fill_pow_table(s_pw, gamma[h], C);
  const float* pw = s_pw;
  const size_t qbase = (size_t(bh) * T + size_t(i) * C) * dk;
  const size_t vbase = (size_t(bh) * T + size_t(i) * C) * dv;
  const float* Pz = P + size_t(z) * C * C;
  const float* Sz = S + size_t(z) * dk * dv;
  float acc[4][4] = {};
  {
    // intra: only columns c <= max row of this tile contribute (P is lower triangular)
    const int klim = min(C, m0 + kTile);
    auto fa = [&](int m, int c) { return (m0 + m < C && c < klim) ? Pz[size_t(m0 + m) * C + c] : 0.f; };
    auto fb = [&](int c, int n) {
      return (n0 + n < dv && c < klim) ? ld_elem<DTYPE>(v, vbase + size_t(c) * dv + n0 + n) : 0.f;
    };
    tile_gemm<true, true>(acc, klim, fa, fb, As, Bs);
  }
  if (i > 0) {  // S_0 == 0
    auto fa = [&](int m, int e) {
      return (m0 + m < C && e < dk)
                 ? ld_elem<DTYPE>(q, qbase + size_t(m0 + m) * dk + e) * pw[m0 + m + 1]
                 : 0.f;
    };
    auto fb = [&](int e, int n) { return (n0 + n < dv && e < dk) ? Sz[size_t(e) * dv + n0 + n] : 0.f; };
    tile_gemm<true, true>(acc, dk, fa, fb, As, Bs);
  }
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    const int r = m0 + ty * 4 + ii;
    if (r >= C) continue;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int f = n0 + tx * 4 + jj;
      if (f < dv) st_elem<DTYPE>(o, vbase + size_t(r) * dv + f, acc[ii][jj] / scale);
    }
  }
}

size_t ffma_scratch_floats(int B, int H, int T, int dk, int dv, int C) {
  const size_t nz = size_t(B) * H * (T / C);
  (void)H;
  return nz * C * C + nz * dk * dv;
}

template <int DTYPE>
int run_ffma(const void* q, const void* k, const void* v, void* o, const float* gamma, int B, int H,
             int T, int dk, int dv, int C, float scale, float* scratch, cudaStream_t st) {
  const int nchunk = T / C;
  const size_t nz = size_t(B) * H * nchunk;
  if (C > kMaxChunk) return CB2_BAD_SHAPE;
  float* P = scratch;
  float* KV = P + nz * C * C;
  const unsigned ct = (C + kTile - 1) / kTile, kt = (dk + kTile - 1) / kTile,
                 vt = (dv + kTile - 1) / kTile;
  chunk_local_kernel<DTYPE><<<dim3(unsigned(nz), ct * ct + kt * vt), kThreads, 0, st>>>(
      q, k, v, gamma, P, KV, H, T, dk, dv, C, int(ct), int(vt));
  CB2_LAUNCH_CHECK();
  const size_t per_chunk = size_t(dk) * dv, total = size_t(B) * H * per_chunk;
  state_scan_kernel<<<unsigned((total + 255) / 256), 256, 0, st>>>(KV, gamma, H, nchunk, C, per_chunk,
                                                                  size_t(B) * H);
  CB2_LAUNCH_CHECK();
  output_kernel<DTYPE><<<dim3(unsigned(nz), ct, vt), kThreads, 0, st>>>(q, v, gamma, P, KV, o, H, T, dk,
                                                                       dv, C, scale);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace

// Entry points for the dispatcher in decayed_chunk.cu.
size_t decayed_ffma_scratch_bytes(int B, int H, int T, int dk, int dv, int C) {
  return ffma_scratch_floats(B, H, T, dk, dv, C) * sizeof(float);
}
int decayed_ffma_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B,
                     int H, int T, int dk, int dv, int C, float scale, int dtype, void* scratch,
                     cudaStream_t st) {
  if (dtype == CB2_BF16)
    return run_ffma<CB2_BF16>(q, k, v, o, gamma, B, H, T, dk, dv, C, scale,
                              static_cast<float*>(scratch), st);
  if (dtype == CB2_F32)
    return run_ffma<CB2_F32>(q, k, v, o, gamma, B, H, T, dk, dv, C, scale,
                             static_cast<float*>(scratch), st);
  return CB2_UNSUPPORTED_DTYPE;
}

}  // namespace cb2
