// Chunked decayed attention in ONE launch for small problems (chunk, dk, dv <= 64;
// a few thousand (batch, head, chunk) units at most): the shapes where the
// three-launch path (decayed_chunk_ffma.cu) spends its time on launch gaps and
// global round trips rather than arithmetic.  The four 64 x 64 x 64 products of a
// chunk run as warp-level TF32 MMAs in three passes (value and truncation
// remainder of both operands: fp32 accuracy, fp32 accumulation): a chunk is one
// tile, so what counts is the latency of a product, and the tile-sized tensor-memory
// pipeline of the large kernels has nothing to amortise its set-up over here (on the
// FMA pipes a product took 2.3-3.6 us, two thirds of the kernel).
//
// CTA = one chunk i of one (batch, head).  It stages Q_i, K_i, V_i in shared
// memory once (as stored: the MMA fragments are read with scalar loads, so no transposed
// copy is needed) and then, entirely from shared memory,
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
// (lab/probes/retnet_baseline_probe.py:77-110) at fp32 accuracy.
#include "common.cuh"

namespace cb2 {
namespace {

constexpr int kT = 64;            // tile edge: chunk, dk, dv <= 64
constexpr int kLd = kT + 4;       // padded leading dimension (floats)
constexpr int kSmallThreads = 256;
constexpr int kArr = kT * kLd;    // floats per staged array
constexpr size_t kSmallSmem = (5 * kArr + kT + 8) * sizeof(float);

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

// What a tf32 operand keeps of an fp32 value (the tensor core ignores the low 13 bits) and what it loses.
__device__ __forceinline__ void tf32_split(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_m16n8k8_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// One warp's 16 x 32 tile (rows m0.., columns n0..: four 8-wide MMA tiles) of acc += A B over kdim
// (a multiple of 8), operands in shared memory with arbitrary strides: A(m,k) = Ap[m*a_m + k*a_k],
// B(k,n) = Bp[k*b_k + n*b_n].  WEIGHTED: row k of B is scaled by wrev[-k] (0 from row wlim on).
// Fragment layout of mma.m16n8k8 (g = lane / 4, t = lane % 4): a = A[g | g+8][t | t+4],
// b = B[t | t+4][g], d = D[g | g+8][2t, 2t+1].  Three passes: lo*hi, hi*lo, hi*hi.
template <bool WEIGHTED>
__device__ __forceinline__ void warp_gemm(float (&acc)[4][4], const float* Ap, int a_m, int a_k, const float* Bp,
                                          int b_k, int b_n, int kdim, const float* wrev, int wlim, int m0,
                                          int n0, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const float* a_lo = Ap + (m0 + g) * a_m + t * a_k;
  const float* b_lo = Bp + t * b_k + (n0 + g) * b_n;
#pragma unroll 2
  for (int k0 = 0; k0 < kdim; k0 += 8) {
    uint32_t ah[4], al[4];
    tf32_split(a_lo[k0 * a_k], ah[0], al[0]);
    tf32_split(a_lo[k0 * a_k + 8 * a_m], ah[1], al[1]);
    tf32_split(a_lo[(k0 + 4) * a_k], ah[2], al[2]);
    tf32_split(a_lo[(k0 + 4) * a_k + 8 * a_m], ah[3], al[3]);
    float w0 = 1.f, w1 = 1.f;
    if (WEIGHTED) {
      const int r0 = k0 + t, r1 = r0 + 4;
      w0 = r0 < wlim ? wrev[-r0] : 0.f;
      w1 = r1 < wlim ? wrev[-r1] : 0.f;
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      uint32_t bh[2], bl[2];
      tf32_split(b_lo[k0 * b_k + nt * 8 * b_n] * w0, bh[0], bl[0]);
      tf32_split(b_lo[(k0 + 4) * b_k + nt * 8 * b_n] * w1, bh[1], bl[1]);
      mma_m16n8k8_tf32(acc[nt], al, bh);
      mma_m16n8k8_tf32(acc[nt], ah, bl);
      mma_m16n8k8_tf32(acc[nt], ah, bh);
    }
  }
}

template <int DTYPE>
__global__ void __launch_bounds__(kSmallThreads)
decayed_small_kernel(const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                     void* __restrict__ o, const float* __restrict__ gamma, float* __restrict__ kv_all,
                     int* __restrict__ flags, int n_bh, int H, int T, int dk, int dv, int C, float inv_scale,
                     int* dev_status) {
  extern __shared__ __align__(16) float sm[];
  float* Qn = sm;               // [r][e]  Q
  float* Kn = Qn + kArr;        // [r][e]  K
  float* Vn = Kn + kArr;        // [c][f]  V
  float* Pn = Vn + kArr;        // [r][c]  P
  float* Ss = Pn + kArr;        // [e][f]  state before this chunk
  float* pw = Ss + kArr;        // g^0 .. g^C
  int* s_ok = reinterpret_cast<int*>(pw + kT + 4);

  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int warp = tid >> 5, lane = tid & 31;
  const int m0 = (warp & 3) * 16, n0 = (warp >> 2) * 32;     // this warp's 16 x 32 tile of every product
  const int fg = lane >> 2, ft = lane & 3;                    // fragment row group / column pair
  const int nchunk = T / C;
  const int i = blockIdx.x / n_bh, bh = blockIdx.x % n_bh;    // chunk-major launch order
  const float g = gamma[bh % H];
  const size_t row0 = size_t(bh) * T + size_t(i) * C;
  const int C8 = (C + 7) & ~7, dk8 = (dk + 7) & ~7;           // reduction lengths in whole MMA steps (tiles are zero-padded)

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
      Qn[r * kLd + e] = qv[u];
      Kn[r * kLd + e] = kv[u];
      Vn[r * kLd + e] = vv[u];
    }
  }
  __syncthreads();

  // KV_i[e][f] = sum_r K[r][e] g^(C-1-r) V[r][f]   -> published for the later chunks of this head
  float* kv_mine = kv_all + (size_t(bh) * nchunk + i) * (kT * kT);
  if (i + 1 < nchunk) {
    float acc[4][4] = {};
    warp_gemm<true>(acc, Kn, 1, kLd, Vn, kLd, 1, C8, pw + (C - 1), C, m0, n0, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float* dst = kv_mine + (m0 + fg) * kT + n0 + nt * 8 + 2 * ft;
      __stcg(reinterpret_cast<float2*>(dst), make_float2(acc[nt][0], acc[nt][1]));
      __stcg(reinterpret_cast<float2*>(dst + 8 * kT), make_float2(acc[nt][2], acc[nt][3]));
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* f = flags + size_t(bh) * nchunk + i;
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(f), "r"(1) : "memory");
    }
  }

  // P = (Q K^T) . tril(g^(r-c))
  {
    float acc[4][4] = {};
    warp_gemm<false>(acc, Qn, kLd, 1, Kn, 1, kLd, dk8, nullptr, 0, m0, n0, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = m0 + fg + 8 * h, c = n0 + nt * 8 + 2 * ft;
        const float p0 = (c <= r && r < C) ? acc[nt][2 * h] * pw[r - c] : 0.f;
        const float p1 = (c + 1 <= r && r < C) ? acc[nt][2 * h + 1] * pw[r - c - 1] : 0.f;
        *reinterpret_cast<float2*>(Pn + r * kLd + c) = make_float2(p0, p1);
      }
    }
  }
  __syncthreads();
  float out[4][4] = {};
  warp_gemm<false>(out, Pn, kLd, 1, Vn, kLd, 1, C8, nullptr, 0, m0, n0, lane);      // O = P V

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
    // Four chunks' loads are issued before their dependent FMAs (eight at a time measured the same).
    constexpr int kBatch = 4;
    const float gC = pw[C];
    float st[4][4] = {};
    const float* kv_head = kv_all + size_t(bh) * nchunk * (kT * kT) + (ty * 4) * kT + tx * 4;
    for (int j0 = 0; j0 < i; j0 += kBatch) {
      float4 x[kBatch][4];
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
          x[u][ii] = (j0 + u < i) ? __ldcg(reinterpret_cast<const float4*>(kv_head + size_t(j0 + u) * (kT * kT) + ii * kT))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (j0 + u < i) {
#pragma unroll
          for (int ii = 0; ii < 4; ++ii) {
            st[ii][0] = fmaf(gC, st[ii][0], x[u][ii].x);
            st[ii][1] = fmaf(gC, st[ii][1], x[u][ii].y);
            st[ii][2] = fmaf(gC, st[ii][2], x[u][ii].z);
            st[ii][3] = fmaf(gC, st[ii][3], x[u][ii].w);
          }
        }
      }
    }
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
      *reinterpret_cast<float4*>(Ss + (ty * 4 + ii) * kLd + tx * 4) =
          make_float4(st[ii][0], st[ii][1], st[ii][2], st[ii][3]);
    __syncthreads();
    float cross[4][4] = {};
    warp_gemm<false>(cross, Qn, kLd, 1, Ss, kLd, 1, dk8, nullptr, 0, m0, n0, lane);   // Q S
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float gr = pw[min(m0 + fg + 8 * h + 1, C)];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        out[nt][2 * h] = fmaf(gr, cross[nt][2 * h], out[nt][2 * h]);
        out[nt][2 * h + 1] = fmaf(gr, cross[nt][2 * h + 1], out[nt][2 * h + 1]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = m0 + fg + 8 * h;
    if (r >= C) continue;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int f = n0 + nt * 8 + 2 * ft;
      if (f < dv) st_e<DTYPE>(o, (row0 + r) * dv + f, out[nt][2 * h] * inv_scale);
      if (f + 1 < dv) st_e<DTYPE>(o, (row0 + r) * dv + f + 1, out[nt][2 * h + 1] * inv_scale);
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
