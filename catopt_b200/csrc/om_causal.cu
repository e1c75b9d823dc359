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
                     int dk, int dv, float scale, int causal, int key_offset, const float* m_in,
                     const float* l_in, const float* a_in, float* m_out, float* l_out, float* a_out,
                     const OmBias& bias, int* dev_status, cudaStream_t st);

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
                 float* __restrict__ a_out, int split_len, const OmBias bias) {
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
  // With split_len > 0 (decode: few queries, many keys) blockIdx.z owns keys
  // [z*split_len, (z+1)*split_len) and writes a partial carrier to slice z of the outputs;
  // the partials are folded afterwards (om_combine_kernel).
  const int k_beg = split_len > 0 ? int(blockIdx.z) * split_len : 0;
  const int k_lim = split_len > 0 ? min(Tk, k_beg + split_len) : Tk;      // keys of this CTA end here
  const int k_end = causal ? max(k_beg, int(min((long long)k_lim, (long long)q0 + kBlk - key_offset))) : k_lim;
  const size_t z_rows = split_len > 0 ? size_t(blockIdx.z) * gridDim.y * Tq : 0;
  for (int k0 = k_beg; k0 < k_end; k0 += kBlk) {
    __syncthreads();  // previous block's Pt / Kt / Vs fully consumed (and Qt written)
    for (int i = tid; i < kBlk * dk; i += kOmThreads) {
      const int c = i / dk, e = i % dk;
      Kt[e * kLd + c] = (k0 + c < k_lim) ? ld_e<DTYPE>(k, kbase + size_t(k0 + c) * dk + e) : 0.f;
    }
    for (int i = tid; i < kBlk * dv; i += kOmThreads) {
      const int c = i / dv, f = i % dv;
      Vs[c * dv + f] = (k0 + c < k_lim) ? ld_e<DTYPE>(v, vbase + size_t(k0 + c) * dv + f) : 0.f;
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
        if ((causal && c + key_offset > t) || c >= k_lim) s[i][j] = -INFINITY;
        else if (bias.p && t < Tq)       // an explicit attention mask in additive form (scores are scaled already)
          s[i][j] += __ldg(bias.p + (bh / bias.H) * bias.sb + (bh % bias.H) * bias.sh + (long long)t * bias.sq + c);
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
    const size_t srow = z_rows + size_t(bh) * Tq + t;
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

// Decode shapes (at most kDecRows query rows, many keys): the step is a stream over
// K and V, so it is laid out for memory bandwidth instead of for tiles.  A warp
// takes 32 keys at a time.  Keys: asynchronous 16-byte copies, coalesced (a copy
// instruction = 128 bytes of four neighbouring rows), into a swizzled shared-memory
// slot, two 128-byte segments of the 32 rows in flight ahead of the one in use (with
// lane = key straight from global memory every load instruction touched 32 cache
// lines, and the L1 tag stage, not DRAM, set the pace: 5.0 TB/s; now 6.5).  Scores:
// lane = key, the lane walks its key's row in the slot in 16-byte pieces against the
// query rows kept in shared memory (no cross-lane traffic).  Softmax: one warp max
// and one warp sum per query row and batch.  Values: lane = four value columns, the
// rows stream in coalesced in register batches (the next batch in flight while one is
// used, the first one already during the scores), the 32 probabilities broadcast one
// by one with a shuffle.  The eight warps of a CTA fold their carriers in shared
// memory and write one partial carrier per key split.
constexpr int kDecRows = 8;
constexpr int kDecWarps = 8;
constexpr int kDecSlot = 32 * 128;   // a warp's key slot: 128 bytes of 32 key rows
constexpr int kDecSmem = kDecWarps * 2 * kDecSlot;   // two slots per warp (>= the carriers of 8 rows x 8 warps)
static_assert(kDecSmem >= kDecWarps * kDecRows * 128 * 4, "the warps' carriers reuse the key slots");
// CTAs per SM the decode kernel is compiled for (registers: two batches of value rows in flight per
// thread plus ROWS carriers; three CTAs would spill) and its key splits are sized for.  One query row
// of bf16 keys, B1 H32 Tk 65536 d128: 165 us at two CTAs per SM, 203 us at three.
__host__ __device__ constexpr int dec_ctas_per_sm(int rows) { return rows <= 4 ? 2 : 1; }

template <int DTYPE>
struct DecLd;
template <>
struct DecLd<CB2_BF16> {
  static constexpr int kPiece = 8;    // elements per 16-byte piece
  __device__ static void piece(const uint4 u, float (&x)[8]) {
    x[0] = bf16lo_to_f32(u.x); x[1] = bf16hi_to_f32(u.x); x[2] = bf16lo_to_f32(u.y); x[3] = bf16hi_to_f32(u.y);
    x[4] = bf16lo_to_f32(u.z); x[5] = bf16hi_to_f32(u.z); x[6] = bf16lo_to_f32(u.w); x[7] = bf16hi_to_f32(u.w);
  }
  // four value columns: loaded raw (kept in registers while in flight), converted at use
  using Raw4 = uint2;
  static constexpr int kValueRows = 16;    // value rows per register batch (32 registers)
  __device__ static Raw4 four_raw(const void* p, size_t i) {
    return __ldcs(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + i));
  }
  __device__ static Raw4 zero_raw() { return make_uint2(0u, 0u); }
  __device__ static void four(const Raw4 u, float (&x)[4]) {
    x[0] = bf16lo_to_f32(u.x); x[1] = bf16hi_to_f32(u.x); x[2] = bf16lo_to_f32(u.y); x[3] = bf16hi_to_f32(u.y);
  }
  __device__ static float one(const void* p, size_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
};
template <>
struct DecLd<CB2_F32> {
  static constexpr int kPiece = 4;
  __device__ static void piece(const uint4 u, float (&x)[4]) {
    x[0] = __uint_as_float(u.x); x[1] = __uint_as_float(u.y); x[2] = __uint_as_float(u.z); x[3] = __uint_as_float(u.w);
  }
  using Raw4 = float4;
  static constexpr int kValueRows = 8;
  __device__ static Raw4 four_raw(const void* p, size_t i) {
    return __ldcs(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i));
  }
  __device__ static Raw4 zero_raw() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ static void four(const Raw4 u, float (&x)[4]) {
    x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w;
  }
  __device__ static float one(const void* p, size_t i) { return static_cast<const float*>(p)[i]; }
};

// dk a multiple of the 16-byte piece (8 bf16 / 4 fp32), dv a multiple of 4, both <= 128;
// Tq <= ROWS (1, 2, 4 or 8).
// BIAS: an additive fp32 mask over this block's keys (-inf hides a key), read through strides.
template <int DTYPE, int ROWS, bool BIAS>
__global__ void __launch_bounds__(kDecWarps * 32, dec_ctas_per_sm(ROWS))
om_decode_kernel(const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v, int Tq,
                 int Tk, int dk, int dv, float scale, int causal, int key_offset, int split_len,
                 float* __restrict__ pm, float* __restrict__ pl, float* __restrict__ pa, const OmBias bias) {
  using L = DecLd<DTYPE>;
  constexpr int P = L::kPiece;
  __shared__ __align__(16) float s_q[ROWS][128];
  __shared__ float s_m[kDecWarps][ROWS], s_l[kDecWarps][ROWS];
  // two 4 KB key slots per warp while the keys stream; the warps' carriers afterwards
  extern __shared__ __align__(128) unsigned char s_buf[];
  float (*s_a)[ROWS][128] = reinterpret_cast<float (*)[ROWS][128]>(s_buf);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* slots = s_buf + warp * (2 * kDecSlot);
  const int bh = blockIdx.y, z = blockIdx.x;
  const int c0 = lane * 4;
  const bool vcol = c0 < dv;
  const int k_beg = z * split_len, k_lim = min(Tk, k_beg + split_len);
  const size_t kbase = size_t(bh) * Tk * dk, vbase = size_t(bh) * Tk * dv;
  for (int x = threadIdx.x; x < ROWS * 128; x += blockDim.x) {
    const int r = x / 128, c = x % 128;
    s_q[r][c] = (r < Tq && c < dk) ? L::one(q, (size_t(bh) * Tq + r) * dk + c) * scale : 0.f;
  }
  __syncthreads();
  float m[ROWS], l[ROWS], a[ROWS][4];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) a[r][e] = 0.f;
  }
  const int npiece = dk / P;
  const int nseg = (npiece + 7) / 8;             // 128-byte segments of a key row
  const size_t rowb = size_t(dk) * (16 / P);     // bytes of a key row
  const unsigned char* kb = static_cast<const unsigned char*>(k) + kbase * (16 / P);
  // Keys come in coalesced and asynchronously: one copy instruction moves 128 bytes of four
  // neighbouring key rows (lane = 16-byte piece), eight instructions one segment of the warp's 32 keys,
  // straight into one of the warp's two shared-memory slots (chunk c of row r at c ^ (r % 8):
  // conflict-free for the copy and for the read-back with lane = key).  Two segments are always in
  // flight ahead of the one being scored.
  const int j_first = k_beg + warp * 32;
  const int nblk = j_first < k_lim ? (k_lim - j_first + kDecWarps * 32 - 1) / (kDecWarps * 32) : 0;
  int is_blk = 0, is_seg = 0, is_n = 0;          // next (block, segment) to copy, and how many were
  auto k_issue = [&]() {
    if (is_blk < nblk) {
      const int pc = is_seg * 8 + (lane & 7);
      if (pc < npiece) {
        const int jb = j_first + is_blk * (kDecWarps * 32);
        unsigned char* dst = slots + (is_n & 1) * kDecSlot;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int row = u * 4 + (lane >> 3);
          const int jr = min(jb + row, k_lim - 1);
          cp_async16(dst + row * 128 + (((lane & 7) ^ (row & 7)) << 4), kb + size_t(jr) * rowb + size_t(pc) * 16);
        }
      }
      if (++is_seg == nseg) { is_seg = 0; ++is_blk; }
    }
    ++is_n;
    cp_async_commit();                            // one group per call, empty past the end
  };
  k_issue();
  k_issue();
  constexpr int kVB = L::kValueRows;
  typename L::Raw4 va[kVB], vb[kVB];
  int use_n = 0;
  for (int j0 = j_first; j0 < k_lim; j0 += kDecWarps * 32) {
    // ---- scores of this lane's key against every query row
    const int j = j0 + lane;
    const bool live = j < k_lim;
    auto v_issue = [&](typename L::Raw4 (&buf)[kVB], int jj0) {
#pragma unroll
      for (int u = 0; u < kVB; ++u) {
        const int jr = min(j0 + jj0 + u, k_lim - 1);
        buf[u] = vcol ? L::four_raw(v, vbase + size_t(jr) * dv + c0) : L::zero_raw();
      }
    };
    float sc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) sc[r] = 0.f;
    for (int seg = 0; seg < nseg; ++seg, ++use_n) {
      cp_async_wait_one();                        // all but the newest group: this segment has landed
      __syncwarp();
      if (seg + 1 == nseg) v_issue(va, 0);        // the first value rows fly during the scores and the softmax
      const unsigned char* slot = slots + (use_n & 1) * kDecSlot;
      const int nc = min(8, npiece - seg * 8);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < nc) {
          float x[P];
          L::piece(*reinterpret_cast<const uint4*>(slot + lane * 128 + ((c ^ (lane & 7)) << 4)), x);
          const int e0 = (seg * 8 + c) * P;
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
#pragma unroll
            for (int e4 = 0; e4 < P; e4 += 4) {
              const float4 qq = *reinterpret_cast<const float4*>(&s_q[r][e0 + e4]);   // broadcast read
              sc[r] = fmaf(qq.x, x[e4], fmaf(qq.y, x[e4 + 1], fmaf(qq.z, x[e4 + 2], fmaf(qq.w, x[e4 + 3], sc[r]))));
            }
          }
        }
      }
      __syncwarp();
      k_issue();                                  // into the slot just read
    }
    // ---- softmax bookkeeping per row: p of this lane's key, running (m, l), rescaled a
    float p[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      bool hidden = !live || r >= Tq || (causal && j + key_offset > r);
      float sv = hidden ? -INFINITY : sc[r];
      if (BIAS && !hidden) {                      // lane = key: one coalesced row of the mask per query row
        sv += __ldg(bias.p + (bh / bias.H) * bias.sb + (bh % bias.H) * bias.sh + (long long)r * bias.sq + j);
        hidden = sv == -INFINITY;
      }
      float mb = sv;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, off));
      const float mn = fmaxf(m[r], mb);
      const float alpha = (m[r] == -INFINITY) ? 0.f : expf(m[r] - mn);
      p[r] = hidden ? 0.f : expf(sv - mn);
      float ps = p[r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
      l[r] = l[r] * alpha + ps;
#pragma unroll
      for (int e = 0; e < 4; ++e) a[r][e] *= alpha;
      m[r] = mn;
    }
    // ---- values: a[r][lane's 4 columns] += sum_jj p_jj[r] * v_jj[columns]; the rows come in register
    // batches, the next batch in flight while one is used (rows past the end repeat the last row: p = 0)
    auto v_use = [&](const typename L::Raw4 (&buf)[kVB], int jj0) {
#pragma unroll
      for (int u = 0; u < kVB; ++u) {
        float vx[4];
        L::four(buf[u], vx);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const float pj = __shfl_sync(0xffffffffu, p[r], jj0 + u);
#pragma unroll
          for (int e = 0; e < 4; ++e) a[r][e] = fmaf(pj, vx[e], a[r][e]);
        }
      }
    };
#pragma unroll
    for (int b = 0; b < 32 / kVB; b += 2) {
      v_issue(vb, (b + 1) * kVB);
      v_use(va, b * kVB);
      if (b + 2 < 32 / kVB) v_issue(va, (b + 2) * kVB);
      v_use(vb, (b + 1) * kVB);
    }
  }
  cp_async_wait_all();
  // fold the eight warps' carriers (in warp order, so the result is deterministic)
  __syncthreads();   // the carriers take the place of the key slots
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    if (lane == 0) {
      s_m[warp][r] = m[r];
      s_l[warp][r] = l[r];
    }
    if (vcol) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s_a[warp][r][c0 + e] = a[r][e];
    }
  }
  __syncthreads();
  const size_t rows = size_t(gridDim.y) * Tq;
  for (int idx = threadIdx.x; idx < Tq * 32; idx += blockDim.x) {
    const int r = idx / 32, ln = idx % 32;
    float mm = -INFINITY;
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, s_m[w][r]);
    float ll = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < kDecWarps; ++w) {
      const float wgt = (s_m[w][r] == -INFINITY) ? 0.f : expf(s_m[w][r] - mm);
      ll += s_l[w][r] * wgt;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (ln * 4 + e < dv) acc[e] += s_a[w][r][ln * 4 + e] * wgt;
    }
    const size_t row = size_t(z) * rows + size_t(bh) * Tq + r;
    if (ln == 0) {
      pm[row] = mm;
      pl[row] = ll;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (ln * 4 + e < dv) pa[row * dv + ln * 4 + e] = acc[e];
  }
}

// Fold the caller's state (optional) and Z partial carriers, in key order, with the
// monoid's compose rule; one warp per query row, lanes over the value columns.
__global__ void om_combine_kernel(const float* __restrict__ m_in, const float* __restrict__ l_in,
                                  const float* __restrict__ a_in, const float* __restrict__ pm,
                                  const float* __restrict__ pl, const float* __restrict__ pa,
                                  float* __restrict__ m_out, float* __restrict__ l_out,
                                  float* __restrict__ a_out, size_t rows, int dv, int Z) {
  const size_t row = (blockIdx.x * size_t(blockDim.x) + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (row >= rows) return;
  float m = m_in ? m_in[row] : -INFINITY, l = m_in ? l_in[row] : 0.f;
  float a[4];   // dv <= 128: four columns per lane
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int f = lane + 32 * u;
    a[u] = (m_in && f < dv) ? a_in[row * dv + f] : 0.f;
  }
  for (int z = 0; z < Z; ++z) {
    const size_t zr = size_t(z) * rows + row;
    const float m2 = pm[zr], l2 = pl[zr];
    const float mn = fmaxf(m, m2);
    // a side that has seen no key (m = -inf) contributes exactly 0
    const float w1 = (m == -INFINITY) ? 0.f : expf(m - mn);
    const float w2 = (m2 == -INFINITY) ? 0.f : expf(m2 - mn);
    l = l * w1 + l2 * w2;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int f = lane + 32 * u;
      if (f < dv) a[u] = a[u] * w1 + pa[zr * dv + f] * w2;
    }
    m = mn;
  }
  if (lane == 0) {
    m_out[row] = m;
    l_out[row] = l;
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int f = lane + 32 * u;
    if (f < dv) a_out[row * dv + f] = a[u];
  }
}

// Key splits of the decode kernel: as many as fit in ONE wave of resident CTAs
// (rounding up would leave a second, nearly empty wave), at least 256 keys each.
int om_decode_splits(int B, int H, int Tq, int Tk) {
  const int rows = Tq <= 1 ? 1 : Tq <= 2 ? 2 : Tq <= 4 ? 4 : 8;
  long long z = (dec_ctas_per_sm(rows) * 148) / ((long long)B * H);
  const long long most = (Tk + 255) / 256;
  if (z > most) z = most;
  if (z > 65535) z = 65535;
  return z < 1 ? 1 : int(z);
}
bool om_decode_shape(int Tq, int Tk, int dk, int dv, int dtype) {
  return Tq <= kDecRows && Tk >= 256 && dk % (dtype == CB2_BF16 ? 8 : 4) == 0 && dv % 4 == 0;
}

// Key splits for a step: only when the query tiles alone leave most SMs idle.
int om_step_splits(int B, int H, int Tq, int Tk) {
  const long long ctas = (long long)((Tq + kBlk - 1) / kBlk) * B * H;
  if (ctas >= 148 || Tk < 4 * kBlk) return 1;
  long long z = (2 * 148 + ctas - 1) / ctas;
  const long long most = (Tk + 2 * kBlk - 1) / (2 * kBlk);      // at least two key blocks per split
  if (z > most) z = most;
  if (z > 65535) z = 65535;
  return z < 2 ? 1 : int(z);
}

// Softmax attention of whole sequences, with or without an additive bias.
int om_fwd_impl(const void* q, const void* k, const void* v, void* o, int B, int H, int Tq, int Tk, int dk, int dv,
                float scale, int causal, int dtype, const OmBias& bias, int* dev_status, void* stream) {
  if (!q || !k || !v || !o) return CB2_NULL_PTR;
  if (B <= 0 || H <= 0 || Tq <= 0 || Tk <= 0 || dk <= 0 || dv <= 0) return CB2_BAD_SHAPE;
  if (dk > kMaxD || dv > kMaxD) return CB2_BAD_SHAPE;
  if (size_t(B) * H > 65535) return CB2_BAD_SHAPE;
  const size_t smem = (size_t(2 * dk) * (kBlk + 4) + size_t(kBlk) * dv + size_t(kBlk) * (kBlk + 4)) * sizeof(float);
  const dim3 grid((Tq + kBlk - 1) / kBlk, B * H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (om_causal_tc_supported(B, H, Tq, Tk, dk, dv, dtype) && scale > 0.f && aligned16(q) && aligned16(k) &&
      aligned16(v) && aligned16(o))
    return om_causal_tc_run(q, k, v, o, B, H, Tq, Tk, dk, dv, scale, causal ? 1 : 0, 0, nullptr, nullptr, nullptr,
                            nullptr, nullptr, nullptr, bias, dev_status, st);
  if (dtype == CB2_BF16) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_BF16><<<grid, kOmThreads, smem, st>>>(q, k, v, o, Tq, Tk, dk, dv, scale, causal ? 1 : 0, 0, nullptr, nullptr, nullptr, nullptr,
                                                               nullptr, nullptr, 0, bias);
  } else if (dtype == CB2_F32) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_F32><<<grid, kOmThreads, smem, st>>>(q, k, v, o, Tq, Tk, dk, dv, scale, causal ? 1 : 0, 0, nullptr, nullptr, nullptr, nullptr,
                                                               nullptr, nullptr, 0, bias);
  } else {
    return CB2_UNSUPPORTED_DTYPE;
  }
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace
}  // namespace cb2

extern "C" int cb2_om_fwd(const void* q, const void* k, const void* v, void* o, int B, int H, int Tq,
                          int Tk, int dk, int dv, float scale, int causal, int dtype, int* dev_status,
                          void* stream) {
  return cb2::om_fwd_impl(q, k, v, o, B, H, Tq, Tk, dk, dv, scale, causal, dtype, cb2::OmBias{nullptr, 0, 0, 0, 1},
                          dev_status, stream);
}

extern "C" int cb2_om_bias_fwd(const void* q, const void* k, const void* v, void* o, const float* bias,
                               long long bias_stride_b, long long bias_stride_h, long long bias_stride_q, int B,
                               int H, int Tq, int Tk, int dk, int dv, float scale, int causal, int dtype,
                               int* dev_status, void* stream) {
  if (!bias) return CB2_NULL_PTR;
  if (bias_stride_b < 0 || bias_stride_h < 0 || bias_stride_q < 0) return CB2_BAD_SHAPE;
  return cb2::om_fwd_impl(q, k, v, o, B, H, Tq, Tk, dk, dv, scale, causal, dtype,
                          cb2::OmBias{bias, bias_stride_b, bias_stride_h, bias_stride_q, H}, dev_status, stream);
}

extern "C" int cb2_om_causal_fwd(const void* q, const void* k, const void* v, void* o, int B, int H,
                                 int Tq, int Tk, int dk, int dv, float scale, int dtype,
                                 int* dev_status, void* stream) {
  return cb2_om_fwd(q, k, v, o, B, H, Tq, Tk, dk, dv, scale, 1, dtype, dev_status, stream);
}

extern "C" size_t cb2_om_step_scratch_bytes(int B, int H, int Tq, int Tk, int dv) {
  if (B <= 0 || H <= 0 || Tq <= 0 || Tk <= 0 || dv <= 0) return 0;
  const int z = Tq <= cb2::kDecRows && Tk >= 256 ? cb2::om_decode_splits(B, H, Tq, Tk) : cb2::om_step_splits(B, H, Tq, Tk);
  return (z > 1 || (Tq <= cb2::kDecRows && Tk >= 256)) ? size_t(z) * B * H * Tq * (size_t(dv) + 2) * sizeof(float) : 0;
}

namespace cb2 {
namespace {
// One streaming step, with or without an additive bias over this block's keys.
int om_step_impl(const void* q, const void* k, const void* v, const float* m_in, const float* l_in,
                 const float* a_in, float* m_out, float* l_out, float* a_out, int B, int H, int Tq, int Tk, int dk,
                 int dv, float scale, int causal, int key_offset, int dtype, const OmBias& bias, void* scratch,
                 size_t scratch_bytes, int* dev_status, void* stream) {
  if (!q || !k || !v || !m_out || !l_out || !a_out) return CB2_NULL_PTR;
  if ((m_in == nullptr) != (l_in == nullptr) || (m_in == nullptr) != (a_in == nullptr)) return CB2_NULL_PTR;
  if (B <= 0 || H <= 0 || Tq <= 0 || Tk <= 0 || dk <= 0 || dv <= 0) return CB2_BAD_SHAPE;
  if (dk > kMaxD || dv > kMaxD || size_t(B) * H > 65535) return CB2_BAD_SHAPE;
  const size_t smem = (size_t(2 * dk) * (kBlk + 4) + size_t(kBlk) * dv + size_t(kBlk) * (kBlk + 4)) * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t rows = size_t(B) * H * Tq;
  // a handful of query rows against many keys: the streaming (memory-bound) kernel
  if (om_decode_shape(Tq, Tk, dk, dv, dtype) && aligned16(q) && aligned16(k) && aligned16(v) && scratch &&
      !(reinterpret_cast<uintptr_t>(scratch) & 15u)) {
    int Zd = om_decode_splits(B, H, Tq, Tk);
    if (scratch_bytes >= size_t(Zd) * rows * (size_t(dv) + 2) * sizeof(float)) {
      const int len = (Tk + Zd - 1) / Zd;
      Zd = (Tk + len - 1) / len;
      float* dm = static_cast<float*>(scratch);
      float* dl = dm + size_t(Zd) * rows;
      float* da = dl + size_t(Zd) * rows;
      const dim3 dgrid(Zd, B * H);
      if (dtype != CB2_BF16 && dtype != CB2_F32) return CB2_UNSUPPORTED_DTYPE;
#define CB2_DECODE_B(DT, R, HAS)                                                                                 \
  do {                                                                                                           \
    if (cudaFuncSetAttribute(om_decode_kernel<DT, R, HAS>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                             kDecSmem) != cudaSuccess)                                                           \
      return CB2_LAUNCH_FAIL;                                                                                    \
    om_decode_kernel<DT, R, HAS><<<dgrid, kDecWarps * 32, kDecSmem, st>>>(                                      \
        q, k, v, Tq, Tk, dk, dv, scale, causal ? 1 : 0, key_offset, len, dm, dl, da, bias);                      \
  } while (0)
#define CB2_DECODE(DT, R)                                                                                        \
  do {                                                                                                           \
    if (bias.p) CB2_DECODE_B(DT, R, true);                                                                       \
    else CB2_DECODE_B(DT, R, false);                                                                             \
  } while (0)
      const bool bf = dtype == CB2_BF16;
      if (Tq == 1) { if (bf) CB2_DECODE(CB2_BF16, 1); else CB2_DECODE(CB2_F32, 1); }
      else if (Tq == 2) { if (bf) CB2_DECODE(CB2_BF16, 2); else CB2_DECODE(CB2_F32, 2); }
      else if (Tq <= 4) { if (bf) CB2_DECODE(CB2_BF16, 4); else CB2_DECODE(CB2_F32, 4); }
      else { if (bf) CB2_DECODE(CB2_BF16, 8); else CB2_DECODE(CB2_F32, 8); }
#undef CB2_DECODE_B
#undef CB2_DECODE
      CB2_LAUNCH_CHECK();
      om_combine_kernel<<<unsigned((rows * 32 + 255) / 256), 256, 0, st>>>(m_in, l_in, a_in, dm, dl, da, m_out,
                                                                          l_out, a_out, rows, dv, Zd);
      CB2_LAUNCH_CHECK();
      return CB2_OK;
    }
  }
  // bf16 with whole query tiles' worth of rows: the tensor-core kernel carries the state
  if (Tq > kDecRows && om_causal_tc_supported(B, H, Tq, Tk, dk, dv, dtype) && scale > 0.f && aligned16(q) &&
      aligned16(k) && aligned16(v) && aligned16(a_out) && (!a_in || aligned16(a_in)))
    return om_causal_tc_run(q, k, v, nullptr, B, H, Tq, Tk, dk, dv, scale, causal ? 1 : 0, key_offset, m_in, l_in,
                            a_in, m_out, l_out, a_out, bias, dev_status, st);
  // few query tiles: cut the keys over extra CTAs, then fold the partial carriers
  int Z = om_step_splits(B, H, Tq, Tk);
  if (Z > 1 && (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 15u) ||
                scratch_bytes < size_t(Z) * rows * (size_t(dv) + 2) * sizeof(float)))
    Z = 1;
  const int split_len = Z > 1 ? ((Tk + Z - 1) / Z + kBlk - 1) / kBlk * kBlk : 0;
  if (Z > 1) Z = (Tk + split_len - 1) / split_len;
  float* pm = static_cast<float*>(scratch);
  float* pl = Z > 1 ? pm + size_t(Z) * rows : nullptr;
  float* pa = Z > 1 ? pl + size_t(Z) * rows : nullptr;
  const dim3 grid((Tq + kBlk - 1) / kBlk, B * H, Z > 1 ? Z : 1);
  const float* mi = Z > 1 ? nullptr : m_in;
  const float* li = Z > 1 ? nullptr : l_in;
  const float* ai = Z > 1 ? nullptr : a_in;
  float* mo = Z > 1 ? pm : m_out;
  float* lo = Z > 1 ? pl : l_out;
  float* ao = Z > 1 ? pa : a_out;
  if (dtype == CB2_BF16) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_BF16><<<grid, kOmThreads, smem, st>>>(q, k, v, nullptr, Tq, Tk, dk, dv, scale, causal ? 1 : 0,
                                                               key_offset, mi, li, ai, mo, lo, ao, split_len, bias);
  } else if (dtype == CB2_F32) {
    if (cudaFuncSetAttribute(om_causal_kernel<CB2_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             int(smem)) != cudaSuccess)
      return CB2_LAUNCH_FAIL;
    om_causal_kernel<CB2_F32><<<grid, kOmThreads, smem, st>>>(q, k, v, nullptr, Tq, Tk, dk, dv, scale, causal ? 1 : 0,
                                                              key_offset, mi, li, ai, mo, lo, ao, split_len, bias);
  } else {
    return CB2_UNSUPPORTED_DTYPE;
  }
  CB2_LAUNCH_CHECK();
  if (Z > 1) {
    const size_t threads = rows * 32;
    om_combine_kernel<<<unsigned((threads + 255) / 256), 256, 0, st>>>(m_in, l_in, a_in, pm, pl, pa, m_out, l_out,
                                                                      a_out, rows, dv, Z);
    CB2_LAUNCH_CHECK();
  }
  return CB2_OK;
}
}  // namespace
}  // namespace cb2

extern "C" int cb2_om_step(const void* q, const void* k, const void* v, const float* m_in, const float* l_in,
                           const float* a_in, float* m_out, float* l_out, float* a_out, int B, int H, int Tq,
                           int Tk, int dk, int dv, float scale, int causal, int key_offset, int dtype,
                           void* scratch, size_t scratch_bytes, int* dev_status, void* stream) {
  return cb2::om_step_impl(q, k, v, m_in, l_in, a_in, m_out, l_out, a_out, B, H, Tq, Tk, dk, dv, scale, causal,
                           key_offset, dtype, cb2::OmBias{nullptr, 0, 0, 0, 1}, scratch, scratch_bytes, dev_status,
                           stream);
}

extern "C" int cb2_om_bias_step(const void* q, const void* k, const void* v, const float* bias,
                                long long bias_stride_b, long long bias_stride_h, long long bias_stride_q,
                                const float* m_in, const float* l_in, const float* a_in, float* m_out, float* l_out,
                                float* a_out, int B, int H, int Tq, int Tk, int dk, int dv, float scale, int causal,
                                int key_offset, int dtype, void* scratch, size_t scratch_bytes, int* dev_status,
                                void* stream) {
  if (!bias) return CB2_NULL_PTR;
  if (bias_stride_b < 0 || bias_stride_h < 0 || bias_stride_q < 0) return CB2_BAD_SHAPE;
  return cb2::om_step_impl(q, k, v, m_in, l_in, a_in, m_out, l_out, a_out, B, H, Tq, Tk, dk, dv, scale, causal,
                           key_offset, dtype, cb2::OmBias{bias, bias_stride_b, bias_stride_h, bias_stride_q, H},
                           scratch, scratch_bytes, dev_status, stream);
}
