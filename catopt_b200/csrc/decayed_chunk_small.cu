// Chunked decayed attention in ONE launch for small problems on the fp32 FMA
// pipes (chunk, dk, dv <= 64; a few thousand (batch, head, chunk) units at most):
// the shapes where the three-launch path (decayed_chunk_ffma.cu) spends its time
// on launch gaps and global round trips rather than arithmetic.
//
// CTA = one chunk i of one (batch, head).  It stages Q_i, K_i, V_i in shared
// memory once and then, entirely from shared memory,
//   KV_i = (K_i . g^(C-1-r))^T V_i        -> global scratch, then a release flag
//   P_i  = (Q_i K_i^T) . tril(g^(r-c))
//   O    = P_i V_i
//   S_i  = sum_{j<i} g^(C (i-1-j)) KV_j   (Horner over j = 0..i-1, the recurrence's own order)
//   O   += diag(g^(r+1)) Q_i S_i ;  o_i = O / scale.
// Every CTA sums the earlier chunks' KV products itself, so there is no serial
// chain across CTAs: a CTA only waits until the KV products of the chunks before
// it are published.  CTAs are launched chunk-major (all heads' chunk 0 first), so
// a CTA's predecessors have lower block indices and are running or finished
// whenever it runs; the wait is bounded and reports through the status word.
// The same arithmetic as the reference's state-carry recurrence
// (lab/probes/retnet_baseline_probe.py:77-110), fp32 throughout.
#include "common.cuh"

namespace cb2 {
namespace {

constexpr int kT = 64;            // tile edge: chunk, dk, dv <= 64
constexpr int kLd = kT + 4;       // padded leading dimension (floats)
constexpr int kSmallThreads = 256;
constexpr int kArr = kT * kLd;    // floats per staged array
constexpr size_t kSmallSmem = (6 * kArr + kT + 8) * sizeof(float);

template <int DTYPE>
__device__ __forceinline__ float ld_e(const void* p, size_t i) {
  if (DTYPE == CB2_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return static_cast<const float*>(p)[i];
}
template <int DTYPE>
__device__ __forceinline__ void st_e(void* p, size_t i, float v) {
  if (DTYPE == CB2_BF16)
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else
    static_cast<float*>(p)[i] = v;
}

// acc[i][j] += sum_k At[k][ty*4+i] * scale_k * B[k][tx*4+j], operands in shared memory.
template <bool SCALED>
__device__ __forceinline__ void smem_gemm(float (&acc)[4][4], const float* At, const float* B, int kdim,
                                          const float* kscale, int ty, int tx) {
#pragma unroll 4
  for (int k = 0; k < kdim; ++k) {
    float4 av = *reinterpret_cast<const float4*>(At + k * kLd + ty * 4);
    const float4 bv = *reinterpret_cast<const float4*>(B + k * kLd + tx * 4);
    if (SCALED) {
      const float w = kscale[k];
      av.x *= w; av.y *= w; av.z *= w; av.w *= w;
    }
    const float a4[4] = {av.x, av.y, av.z, av.w};
    const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
  }
}

template <int DTYPE>
__global__ void __launch_bounds__(kSmallThreads)
decayed_small_kernel(const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                     void* __restrict__ o, const float* __restrict__ gamma, float* __restrict__ kv_all,
                     int* __restrict__ flags, int n_bh, int H, int T, int dk, int dv, int C, float inv_scale,
                     int* dev_status) {
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm;               // [e][r]  Q transposed
  float* Kt = Qt + kArr;        // [e][c]  K transposed
  float* Kn = Kt + kArr;        // [r][e]  K as stored
  float* Vn = Kn + kArr;        // [c][f]  V as stored
  float* Pt = Vn + kArr;        // [c][r]  P transposed
  float* Ss = Pt + kArr;        // [e][f]  state before this chunk
  float* pw = Ss + kArr;        // g^0 .. g^C
  int* s_ok = reinterpret_cast<int*>(pw + kT + 4);

  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int nchunk = T / C;
  const int i = blockIdx.x / n_bh, bh = blockIdx.x % n_bh;    // chunk-major launch order
  const float g = gamma[bh % H];
  const size_t row0 = size_t(bh) * T + size_t(i) * C;

  for (int x = tid; x <= C; x += kSmallThreads) pw[x] = powf(g, float(x));
  // stage the three tiles, zero-padded to 64 x 64: all of a thread's loads are issued
  // before any is used, so their latencies overlap
  {
    constexpr int kPer = kT * kT / kSmallThreads;   // 16 elements of each tile per thread
    float qv[kPer], kv[kPer], vv[kPer];
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int x = tid + u * kSmallThreads, r = x / kT, e = x % kT;
      const bool in_r = r < C;
      qv[u] = (in_r && e < dk) ? ld_e<DTYPE>(q, (row0 + r) * dk + e) : 0.f;
      kv[u] = (in_r && e < dk) ? ld_e<DTYPE>(k, (row0 + r) * dk + e) : 0.f;
      vv[u] = (in_r && e < dv) ? ld_e<DTYPE>(v, (row0 + r) * dv + e) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int x = tid + u * kSmallThreads, r = x / kT, e = x % kT;
      Qt[e * kLd + r] = qv[u];
      Kt[e * kLd + r] = kv[u];
      Kn[r * kLd + e] = kv[u];
      Vn[r * kLd + e] = vv[u];
    }
  }
  __syncthreads();

  // KV_i[e][f] = sum_r K[r][e] g^(C-1-r) V[r][f]   -> published for the later chunks of this head
  float* kv_mine = kv_all + (size_t(bh) * nchunk + i) * (kT * kT);
  if (i + 1 < nchunk) {
    float acc[4][4] = {};
    // per-row weights g^(C-1-r), reusing Ss as scratch for the reversed table
    for (int x = tid; x < kT; x += kSmallThreads) Ss[x] = x < C ? pw[C - 1 - x] : 0.f;
    __syncthreads();
    smem_gemm<true>(acc, Kn, Vn, C, Ss, ty, tx);
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
      __stcg(reinterpret_cast<float4*>(kv_mine + (ty * 4 + ii) * kT + tx * 4),
             make_float4(acc[ii][0], acc[ii][1], acc[ii][2], acc[ii][3]));
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* f = flags + size_t(bh) * nchunk + i;
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(f), "r"(1) : "memory");
    }
  }

  // P = (Q K^T) . tril(g^(r-c)), kept transposed for the next product
  {
    float acc[4][4] = {};
    smem_gemm<false>(acc, Qt, Kt, dk, nullptr, ty, tx);
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int r = ty * 4 + ii;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int c = tx * 4 + jj;
        Pt[c * kLd + r] = (c <= r && r < C) ? acc[ii][jj] * pw[r - c] : 0.f;
      }
    }
  }
  __syncthreads();
  float out[4][4] = {};
  smem_gemm<false>(out, Pt, Vn, C, nullptr, ty, tx);      // O = P V

  if (i > 0) {
    // wait (bounded) until every earlier chunk of this head has published its KV: lane j of
    // the first warp watches chunk j (at most 32 chunks), so the polls overlap
    if (tid < 32) {
      int ok = 1;
      if (tid < i) {
        const int* f = flags + size_t(bh) * nchunk + tid;
        const WaitBudget budget(kDefaultWaitNs);
        for (uint32_t it = 0;; ++it) {
          int val;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(val) : "l"(f) : "memory");
          if (val != 0) break;
          if ((it & 63u) == 63u) {
            if (budget.spent(it)) { ok = 0; break; }
            __nanosleep(100);
          }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (tid == 0) *s_ok = ok;
    }
    __syncthreads();
    if (!*s_ok) {
      if (tid == 0 && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT);
      return;
    }
    // S_i = sum_j g^(C (i-1-j)) KV_j, Horner in chunk order; this thread's 4 x 4 block.
    // Four chunks' loads are issued before their dependent FMAs.
    const float gC = pw[C];
    float s[4][4] = {};
    const float* kv_head = kv_all + size_t(bh) * nchunk * (kT * kT) + (ty * 4) * kT + tx * 4;
    for (int j0 = 0; j0 < i; j0 += 4) {
      float4 x[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
          x[u][ii] = (j0 + u < i) ? __ldcg(reinterpret_cast<const float4*>(kv_head + size_t(j0 + u) * (kT * kT) + ii * kT))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (j0 + u < i) {
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            s[ii][0] = fmaf(gC, s[ii][0], x[u][ii].x);
            s[ii][1] = fmaf(gC, s[ii][1], x[u][ii].y);
            s[ii][2] = fmaf(gC, s[ii][2], x[u][ii].z);
            s[ii][3] = fmaf(gC, s[ii][3], x[u][ii].w);
          }
        }
      }
    }
    __syncthreads();   // Ss was used as the weight table above
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
      *reinterpret_cast<float4*>(Ss + (ty * 4 + ii) * kLd + tx * 4) =
          make_float4(s[ii][0], s[ii][1], s[ii][2], s[ii][3]);
    __syncthreads();
    float cross[4][4] = {};
    smem_gemm<false>(cross, Qt, Ss, dk, nullptr, ty, tx);   // Q S
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const float gr = pw[min(ty * 4 + ii + 1, C)];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) out[ii][jj] = fmaf(gr, cross[ii][jj], out[ii][jj]);
    }
  }
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    const int r = ty * 4 + ii;
    if (r >= C) continue;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int f = tx * 4 + jj;
      if (f < dv) st_e<DTYPE>(o, (row0 + r) * dv + f, out[ii][jj] * inv_scale);
    }
  }
}

}  // namespace

// Shapes the one-launch kernel takes; scratch is the three-launch path's (its P
// region holds the flags, its KV region the published 64 x 64 products).
bool decayed_small_supported(int B, int H, int T, int dk, int dv, int C) {
  const long long nz = (long long)B * H * (T / C);
  return C <= kT && dk <= kT && dv <= kT && T / C <= 32 && nz <= 4096;
}
size_t decayed_small_scratch_bytes(int B, int H, int T, int C) {
  const size_t nz = size_t(B) * H * (T / C);
  return nz * (size_t(kT) * kT * sizeof(float) + sizeof(int)) + 16;
}

int decayed_small_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B, int H,
                      int T, int dk, int dv, int C, float scale, int dtype, void* scratch, int* dev_status,
                      cudaStream_t st) {
  const int n_bh = B * H, nchunk = T / C;
  const size_t nz = size_t(n_bh) * nchunk;
  float* kv_all = static_cast<float*>(scratch);
  int* flags = reinterpret_cast<int*>(kv_all + nz * kT * kT);
  if (cudaMemsetAsync(flags, 0, nz * sizeof(int), st) != cudaSuccess) return CB2_LAUNCH_FAIL;
  const float inv_scale = 1.0f / scale;
  if (dtype == CB2_F32) {
    if (cudaFuncSetAttribute(decayed_small_kernel<CB2_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(kSmallSmem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    decayed_small_kernel<CB2_F32><<<unsigned(nz), kSmallThreads, kSmallSmem, st>>>(
        q, k, v, o, gamma, kv_all, flags, n_bh, H, T, dk, dv, C, inv_scale, dev_status);
  } else if (dtype == CB2_BF16) {
    if (cudaFuncSetAttribute(decayed_small_kernel<CB2_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(kSmallSmem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    decayed_small_kernel<CB2_BF16><<<unsigned(nz), kSmallThreads, kSmallSmem, st>>>(
        q, k, v, o, gamma, kv_all, flags, n_bh, H, T, dk, dv, C, inv_scale, dev_status);
  } else {
    return CB2_UNSUPPORTED_DTYPE;
  }
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
