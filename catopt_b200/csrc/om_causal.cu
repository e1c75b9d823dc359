// Causal softmax attention through the online-softmax monoid:
//   o_t = sum_{j<=t} softmax_j(scale * q_t.k_j) v_j
// evaluated key block by key block with the running (max, sum, weighted sum)
// triple — the value of the reference's `om_apply(om_compose(...om_elem...))`
// carrier (catopt_torch/torch_bridge.py:1974-2006: `_om_elem`, `_om_compose`;
// read-out a/l at 1887-1890) with its causal mask `cmask` = strict upper
// triangle (catopt_carriers/om.py:1023-1029), i.e. key j is hidden from query t
// when j > t.  A block that is entirely masked contributes nothing (the
// reference's isfinite guard); a row with no visible key at all ends as 0/0 =
// NaN, like dense softmax.
//
// This file: fp32 arithmetic on the FMA pipes, used for fp32 tensors and for
// bf16 shapes the tensor-core kernel (om_causal_tc.cu) does not take.  CTA = 64 queries
// of one (batch, head); key blocks of 64 up to the diagonal; each thread owns a
// 4x4 patch of the 64x64 score block and 4 x (dv/16) output accumulators.
#include "common.cuh"

namespace cb2 {
// tensor-core kernel for bf16 tensors (om_causal_tc.cu)
bool om_causal_tc_supported(int B, int H, int Tq, int Tk, int dk, int dv, int dtype);
int om_causal_tc_run(const void* q, const void* k, const void* v, void* o, int B, int H, int Tq, int Tk,
                     int dk, int dv, float scale, int causal, int* dev_status, cudaStream_t st);

namespace {

constexpr int kBlk = 64;
constexpr int kOmThreads = 256;
constexpr int kMaxD = 128;

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

// shared memory (floats): Qt[dk][68] | Kt[dk][68] | Vs[64][dv] | Pt[64][68]
template <int DTYPE>
__global__ void __launch_bounds__(kOmThreads)
om_causal_kernel(const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v,
                 void* __restrict__ o, int Tq, int Tk, int dk, int dv, float scale, int causal,
                 int key_offset, const float* __restrict__ m_in, const float* __restrict__ l_in,
                 const float* __restrict__ a_in, float* __restrict__ m_out, float* __restrict__ l_out,
                 float* __restrict__ a_out) {
  extern __shared__ __align__(16) float sm[];
  constexpr int kLd = kBlk + 4;
  float* Qt = sm;
  float* Kt = Qt + dk * kLd;
  float* Vs = Kt + dk * kLd;
  float* Pt = Vs + kBlk * dv;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int bh = blockIdx.y, q0 = blockIdx.x * kBlk;
  const size_t qbase = size_t(bh) * Tq * dk, kbase = size_t(bh) * Tk * dk, vbase = size_t(bh) * Tk * dv;
  const int nf = (dv + 63) / 64;  // 64-wide output column groups per thread

  for (int i = tid; i < kBlk * dk; i += kOmThreads) {
    const int r = i / dk, e = i % dk;
    Qt[e * kLd + r] = (q0 + r < Tq) ? ld_e<DTYPE>(q, qbase + size_t(q0 + r) * dk + e) * scale : 0.f;
  }
  // running carrier (m, l, a) per row: the identity (-inf, 0, 0), or the caller's state
  float m_run[4], l_run[4], acc[4][2][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = q0 + ty * 4 + i;
    const bool have = m_in != nullptr && t < Tq;
    const size_t srow = size_t(bh) * Tq + (have ? t : 0);
    m_run[i] = have ? m_in[srow] : -INFINITY;
    l_run[i] = have ? l_in[srow] : 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int f = h * 64 + tx * 4 + j;
        acc[i][h][j] = (have && h < nf && f < dv) ? a_in[srow * dv + f] : 0.f;
      }
  }
  // causal: key j of this call is key (key_offset + j) of the whole sequence and is hidden
  // from query t when key_offset + j > t; blocks past the last query's horizon are skipped
  const int k_end = causal ? max(0, min(Tk, q0 + kBlk - key_offset)) : Tk;
  for (int k0 = 0; k0 < k_end; k0 += kBlk) {
    __syncthreads();  // previous block's Pt / Kt / Vs fully consumed (and Qt written)
    for (int i = tid; i < kBlk * dk; i += kOmThreads) {
      const int c = i / dk, e = i % dk;
      Kt[e * kLd + c] = (k0 + c < Tk) ? ld_e<DTYPE>(k, kbase + size_t(k0 + c) * dk + e) : 0.f;
    }
    for (int i = tid; i < kBlk * dv; i += kOmThreads) {
      const int c = i / dv, f = i % dv;
      Vs[c * dv + f] = (k0 + c < Tk) ? ld_e<DTYPE>(v, vbase + size_t(k0 + c) * dv + f) : 0.f;
    }
    __syncthreads();
    // scores of this thread's 4x4 patch
    float s[4][4] = {};
    for (int e = 0; e < dk; ++e) {
      const float4 qa = *reinterpret_cast<const float4*>(&Qt[e * kLd + ty * 4]);
      const float4 kb = *reinterpret_cast<const float4*>(&Kt[e * kLd + tx * 4]);
      const float a4[4] = {qa.x, qa.y, qa.z, qa.w}, b4[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = fmaf(a4[i], b4[j], s[i][j]);
    }
    // mask, running max / sum per row (a row lives on the 16 lanes sharing ty)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = q0 + ty * 4 + i;
      float mb = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = k0 + tx * 4 + j;
        if ((causal && c + key_offset > t) || c >= Tk) s[i][j] = -INFINITY;
        mb = fmaxf(mb, s[i][j]);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, off));
      const float m_new = fmaxf(m_run[i], mb);
      // a block (or history) that is entirely masked contributes exactly 0
      const float alpha = (m_run[i] == -INFINITY) ? 0.f : expf(m_run[i] - m_new);
      float ps = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s[i][j] = (s[i][j] == -INFINITY) ? 0.f : expf(s[i][j] - m_new);
        ps += s[i][j];
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
      l_run[i] = l_run[i] * alpha + ps;
      m_run[i] = m_new;
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][h][j] *= alpha;
#pragma unroll
      for (int j = 0; j < 4; ++j) Pt[(tx * 4 + j) * kLd + ty * 4 + i] = s[i][j];
    }
    __syncthreads();
    // acc += P . V
    for (int c = 0; c < kBlk; ++c) {
      const float4 pa = *reinterpret_cast<const float4*>(&Pt[c * kLd + ty * 4]);
      const float a4[4] = {pa.x, pa.y, pa.z, pa.w};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h < nf) {
          const int f = h * 64 + tx * 4;
          float b4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) b4[j] = (f + j < dv) ? Vs[c * dv + f + j] : 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][h][j] = fmaf(a4[i], b4[j], acc[i][h][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = q0 + ty * 4 + i;
    if (t >= Tq) continue;
    const size_t srow = size_t(bh) * Tq + t;
    if (m_out != nullptr && tx == 0) {
      m_out[srow] = m_run[i];
      l_out[srow] = l_run[i];
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int f = h * 64 + tx * 4 + j;
        if (h < nf && f < dv) {
          if (m_out != nullptr)
            a_out[srow * dv + f] = acc[i][h][j];                        // the raw carrier
          else
            st_e<DTYPE>(o, srow * dv + f, acc[i][h][j] / l_run[i]);     // the om_apply readout a / l
        }
      }
  }
}

}  // namespace
}  // namespace cb2

extern "C" int cb2_om_fwd(const void* q, const void* k, const void* v, void* o, int B, int H, int Tq,
                          int Tk, int dk, int dv, float scale, int causal, int dtype, int* dev_status,
                          void* stream) {
  using namespace cb2;
  if (!q || !k || !v || !o) return CB2_NULL_PTR;
  if (B <= 0 || H <= 0 || Tq <= 0 || Tk <= 0 || dk <= 0 || dv <= 0) return CB2_BAD_SHAPE;
  if (dk > kMaxD || dv > kMaxD) return CB2_BAD_SHAPE;
  if (size_t(B) * H > 65535) return CB2_BAD_SHAPE;
  const size_t smem = (size_t(2 * dk) * (kBlk + 4) + size_t(kBlk) * dv + size_t(kBlk) * (kBlk + 4)) * sizeof(float);
  const dim3 grid((Tq + kBlk - 1) / kBlk, B * H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (om_causal_tc_supported(B, H, Tq, Tk, dk, dv, dtype) && scale > 0.f && aligned16(q) && aligned16(k) &&
      aligned16(v) && aligned16(o))
    return om_causal_tc_run(q, k, v, o, B, H, Tq, Tk, dk, dv, scale, causal ? 1 : 0, dev_status, st);
  if (dtype == CB2_BF16) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_BF16><<<grid, kOmThreads, smem, st>>>(q, k, v, o, Tq, Tk, dk, dv, scale, causal ? 1 : 0, 0, nullptr, nullptr, nullptr, nullptr,
                                                               nullptr, nullptr);
  } else if (dtype == CB2_F32) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_F32><<<grid, kOmThreads, smem, st>>>(q, k, v, o, Tq, Tk, dk, dv, scale, causal ? 1 : 0, 0, nullptr, nullptr, nullptr, nullptr,
                                                               nullptr, nullptr);
  } else {
    return CB2_UNSUPPORTED_DTYPE;
  }
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

extern "C" int cb2_om_causal_fwd(const void* q, const void* k, const void* v, void* o, int B, int H,
                                 int Tq, int Tk, int dk, int dv, float scale, int dtype,
                                 int* dev_status, void* stream) {
  return cb2_om_fwd(q, k, v, o, B, H, Tq, Tk, dk, dv, scale, 1, dtype, dev_status, stream);
}

extern "C" int cb2_om_step(const void* q, const void* k, const void* v, const float* m_in, const float* l_in,
                           const float* a_in, float* m_out, float* l_out, float* a_out, int B, int H, int Tq,
                           int Tk, int dk, int dv, float scale, int causal, int key_offset, int dtype,
                           void* stream) {
  using namespace cb2;
  if (!q || !k || !v || !m_out || !l_out || !a_out) return CB2_NULL_PTR;
  if ((m_in == nullptr) != (l_in == nullptr) || (m_in == nullptr) != (a_in == nullptr)) return CB2_NULL_PTR;
  if (B <= 0 || H <= 0 || Tq <= 0 || Tk <= 0 || dk <= 0 || dv <= 0 || key_offset < 0) return CB2_BAD_SHAPE;
  if (dk > kMaxD || dv > kMaxD || size_t(B) * H > 65535) return CB2_BAD_SHAPE;
  const size_t smem = (size_t(2 * dk) * (kBlk + 4) + size_t(kBlk) * dv + size_t(kBlk) * (kBlk + 4)) * sizeof(float);
  const dim3 grid((Tq + kBlk - 1) / kBlk, B * H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_BF16) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_BF16><<<grid, kOmThreads, smem, st>>>(q, k, v, nullptr, Tq, Tk, dk, dv, scale, causal ? 1 : 0,
                                                               key_offset, m_in, l_in, a_in, m_out, l_out, a_out);
  } else if (dtype == CB2_F32) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_F32><<<grid, kOmThreads, smem, st>>>(q, k, v, nullptr, Tq, Tk, dk, dv, scale, causal ? 1 : 0,
                                                              key_offset, m_in, l_in, a_in, m_out, l_out, a_out);
  } else {
    return CB2_UNSUPPORTED_DTYPE;
  }
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}
