// Final state of a diagonal scan from its leaf maps, without re-ordering them:
//     out = a_root * h + b_root,   (a_root, b_root) = f_0 . f_1 . ... . f_{n-1},
// f_j(h) = a_j*h + b_j, leaves stored in PRODUCT order (f_0 is the latest step),
// the order in which the reference stacks them for `fused_diag_levels`
// (catopt_carriers/scan_fused.py:100-120) inside
// `BatchedScanModule._forward_fused` (scan_lower.py:785-807).
//
// The reference halves the leaf stack log2(n) times (two kernels per level,
// about twice the leaf bytes of traffic).  Composition is associative, so the
// same map comes out of ONE pass in stored order with the recurrence
//     B += A * b_j ;  A *= a_j          (A = 1, B = 0 at the start)
// per state element: the leaves are read once, nothing is flipped or copied.
// HBM-bound streaming: a thread owns 16 bytes of the state row and walks n with
// eight steps of loads in flight; when the state alone gives too few threads to
// fill the GPU, n is cut into segments whose partial maps (fp32, in caller
// scratch) a second small kernel folds in order and applies to h.
#include "common.cuh"

namespace cb2 {
namespace {

constexpr int kComposeThreads = 256;
constexpr int kUnroll = 8;

template <int DTYPE>
struct Vec;
template <>
struct Vec<CB2_F32> {
  static constexpr int kElems = 4;
  __device__ static void ld(const void* p, size_t i, float (&v)[4]) {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i));
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  __device__ static float ld1(const void* p, size_t i) { return __ldcs(static_cast<const float*>(p) + i); }
  __device__ static void st1(void* p, size_t i, float v) { static_cast<float*>(p)[i] = v; }
  __device__ static void st(void* p, size_t i, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4*>(static_cast<float*>(p) + i), make_float4(v[0], v[1], v[2], v[3]));
  }
};
template <>
struct Vec<CB2_BF16> {
  static constexpr int kElems = 8;
  __device__ static void ld(const void* p, size_t i, float (&v)[8]) {
    const uint4 x = __ldcs(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p) + i));
    v[0] = bf16lo_to_f32(x.x); v[1] = bf16hi_to_f32(x.x);
    v[2] = bf16lo_to_f32(x.y); v[3] = bf16hi_to_f32(x.y);
    v[4] = bf16lo_to_f32(x.z); v[5] = bf16hi_to_f32(x.z);
    v[6] = bf16lo_to_f32(x.w); v[7] = bf16hi_to_f32(x.w);
  }
  __device__ static float ld1(const void* p, size_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
  __device__ static void st1(void* p, size_t i, float v) {
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  }
  __device__ static void st(void* p, size_t i, const float (&v)[8]) {
    __stcs(reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p) + i),
           make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                      pack_bf16x2(v[6], v[7])));
  }
};

// Partial map of leaves [j0, j1) for the state elements of this thread.
// VEC: 16-byte vector loads (S a multiple of the vector width, aligned rows).
// CHRONO: the rows are stored in time order (row 0 = first step) instead of product
// order; the partial map then grows on the left, B = a_j*B + b_j.
// a_stride / b_stride: elements between consecutive rows (S, or 0 for a row shared by
// every step).
template <int DTYPE, bool VEC, bool CHRONO>
__global__ void __launch_bounds__(kComposeThreads)
compose_partial_kernel(const void* __restrict__ a, const void* __restrict__ b, long long n, long long S,
                       long long seg_len, float* __restrict__ part_a, float* __restrict__ part_b,
                       long long a_stride, long long b_stride) {
  using V = Vec<DTYPE>;
  constexpr int E = VEC ? V::kElems : 1;
  const long long c0 = (blockIdx.x * (long long)kComposeThreads + threadIdx.x) * E;
  if (c0 >= S) return;
  const long long j0 = blockIdx.y * seg_len;
  const long long j1 = j0 + seg_len < n ? j0 + seg_len : n;
  float A[E], B[E];
#pragma unroll
  for (int e = 0; e < E; ++e) { A[e] = 1.f; B[e] = 0.f; }
  long long j = j0;
  for (; j + kUnroll <= j1; j += kUnroll) {
    float av[kUnroll][E], bv[kUnroll][E];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const size_t offa = size_t(j + u) * size_t(a_stride) + size_t(c0);
      const size_t offb = size_t(j + u) * size_t(b_stride) + size_t(c0);
      if constexpr (VEC) {
        V::ld(a, offa, av[u]);
        V::ld(b, offb, bv[u]);
      } else {
        av[u][0] = V::ld1(a, offa);
        bv[u][0] = V::ld1(b, offb);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        if constexpr (CHRONO) {
          B[e] = fmaf(av[u][e], B[e], bv[u][e]);
        } else {
          B[e] = fmaf(A[e], bv[u][e], B[e]);
        }
        A[e] *= av[u][e];
      }
  }
  for (; j < j1; ++j) {
    const size_t offa = size_t(j) * size_t(a_stride) + size_t(c0);
    const size_t offb = size_t(j) * size_t(b_stride) + size_t(c0);
    float av[E], bv[E];
    if constexpr (VEC) {
      V::ld(a, offa, av);
      V::ld(b, offb, bv);
    } else {
      av[0] = V::ld1(a, offa);
      bv[0] = V::ld1(b, offb);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if constexpr (CHRONO) {
        B[e] = fmaf(av[e], B[e], bv[e]);
      } else {
        B[e] = fmaf(A[e], bv[e], B[e]);
      }
      A[e] *= av[e];
    }
  }
  const size_t base = size_t(blockIdx.y) * size_t(S) + size_t(c0);
#pragma unroll
  for (int e = 0; e < E; ++e) {
    part_a[base + e] = A[e];
    part_b[base + e] = B[e];
  }
}

// Fold the segment maps in order (segment 0 holds the latest steps, or with chrono
// the earliest) and apply to h.
template <int DTYPE>
__global__ void __launch_bounds__(kComposeThreads)
compose_apply_kernel(const float* __restrict__ part_a, const float* __restrict__ part_b,
                     const void* __restrict__ h, void* __restrict__ out, int nseg, long long S, int chrono) {
  using V = Vec<DTYPE>;
  const long long c = blockIdx.x * (long long)kComposeThreads + threadIdx.x;
  if (c >= S) return;
  float A = 1.f, B = 0.f;
  for (int s = 0; s < nseg; ++s) {
    const size_t i = size_t(s) * size_t(S) + size_t(c);
    B = chrono ? fmaf(part_a[i], B, part_b[i]) : fmaf(A, part_b[i], B);
    A *= part_a[i];
  }
  V::st1(out, size_t(c), fmaf(A, V::ld1(h, size_t(c)), B));
}

// All prefix maps of rows in time order, one pass: Pa[t] = a_t * Pa[t-1], Pb[t] = a_t * Pb[t-1] + b_t
// (Pa[-1] = 1, Pb[-1] = 0), both written for every step.  A thread owns 16 bytes of the state row
// and walks the steps with eight steps of loads in flight; fp32 running maps, rounded on store.
// When the state alone gives too few threads, the steps are cut into segments (blockIdx.y): the
// segments' total maps come from compose_partial_kernel<CHRONO> first, and a segment starts from
// the fold of the totals before it instead of the identity (a and b are then read twice).
// STATES: the same walk started from an initial state h0 instead of the identity map, storing
// only the running state (pb = every h_t; pa is not touched): 3 units of traffic per step.
template <int DTYPE, bool VEC, bool STATES>
__global__ void __launch_bounds__(128)
prefix_maps_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ pa,
                   void* __restrict__ pb, long long n, long long S, long long a_stride, long long b_stride,
                   long long seg_len, const float* __restrict__ part_a, const float* __restrict__ part_b,
                   const void* __restrict__ h0) {
  using V = Vec<DTYPE>;
  constexpr int E = VEC ? V::kElems : 1;
  const long long c0 = (blockIdx.x * 128ll + threadIdx.x) * E;
  if (c0 >= S) return;
  const long long j0 = blockIdx.y * seg_len;
  n = j0 + seg_len < n ? j0 + seg_len : n;     // this segment's steps are [j0, n)
  float A[E], B[E];
#pragma unroll
  for (int e = 0; e < E; ++e) { A[e] = 1.f; B[e] = STATES ? V::ld1(h0, size_t(c0) + e) : 0.f; }
  for (unsigned sgm = 0; sgm < blockIdx.y; ++sgm) {
    const size_t i = size_t(sgm) * size_t(S) + size_t(c0);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      B[e] = fmaf(part_a[i + e], B[e], part_b[i + e]);
      A[e] *= part_a[i + e];
    }
  }
  auto step = [&](const float (&av)[E], const float (&bv)[E], long long j) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      B[e] = fmaf(av[e], B[e], bv[e]);
      A[e] *= av[e];
    }
    const size_t off = size_t(j) * size_t(S) + size_t(c0);
    if constexpr (VEC) {
      if constexpr (!STATES) V::st(pa, off, A);
      V::st(pb, off, B);
    } else {
      if constexpr (!STATES) V::st1(pa, off, A[0]);
      V::st1(pb, off, B[0]);
    }
  };
  long long j = j0;
  for (; j + kUnroll <= n; j += kUnroll) {
    float av[kUnroll][E], bv[kUnroll][E];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const size_t offa = size_t(j + u) * size_t(a_stride) + size_t(c0);
      const size_t offb = size_t(j + u) * size_t(b_stride) + size_t(c0);
      if constexpr (VEC) {
        V::ld(a, offa, av[u]);
        V::ld(b, offb, bv[u]);
      } else {
        av[u][0] = V::ld1(a, offa);
        bv[u][0] = V::ld1(b, offb);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) step(av[u], bv[u], j + u);
  }
  for (; j < n; ++j) {
    float av[E], bv[E];
    const size_t offa = size_t(j) * size_t(a_stride) + size_t(c0);
    const size_t offb = size_t(j) * size_t(b_stride) + size_t(c0);
    if constexpr (VEC) {
      V::ld(a, offa, av);
      V::ld(b, offb, bv);
    } else {
      av[0] = V::ld1(a, offa);
      bv[0] = V::ld1(b, offb);
    }
    step(av, bv, j);
  }
}

// Segments for the all-prefix pass: enough CTAs of 128 threads for about eight per SM,
// at least 64 steps per segment; 1 = plain single pass.  Segments cost a second read of a
// and b (6 units of traffic instead of 4), which pays only while one pass would leave most
// SMs idle: measured, 64 CTAs stream 3.4 TB/s in one pass and 4.0 TB/s segmented, 128 CTAs
// 4.05 against 3.8.
int prefix_segments(long long n, long long S, int elems_per_thread) {
  long long ctas = (S / elems_per_thread + 127) / 128;
  if (ctas < 1) ctas = 1;
  if (ctas >= 96) return 1;
  long long want = (8 * 148 + ctas - 1) / ctas;
  const long long most = n / 64 > 0 ? n / 64 : 1;
  if (want > most) want = most;
  if (want < 1) want = 1;
  if (want > 65535) want = 65535;
  return int(want);
}

template <int DTYPE, bool STATES = false>
int run_prefix(const void* a, const void* b, void* pa, void* pb, long long n, long long S, long long a_stride,
               long long b_stride, void* scratch, size_t scratch_bytes, cudaStream_t st, const void* h0 = nullptr) {
  using V = Vec<DTYPE>;
  const bool vec = S % V::kElems == 0 && aligned16(a) && aligned16(b) && (STATES || aligned16(pa)) && aligned16(pb);
  const int E = vec ? V::kElems : 1;
  const long long threads = S / E;
  const long long blocks = (threads + 127) / 128;
  if (blocks > 0x7fffffffll) return CB2_BAD_SHAPE;
  int nseg = prefix_segments(n, S, E);
  if (nseg > 1 && (!scratch || !aligned16(scratch) || scratch_bytes < size_t(2) * nseg * size_t(S) * sizeof(float)))
    nseg = 1;   // no room for the segment totals: one pass over all steps per thread
  const long long seg_len = (n + nseg - 1) / nseg;
  float* part_a = static_cast<float*>(scratch);
  float* part_b = nseg > 1 ? part_a + size_t(nseg) * size_t(S) : nullptr;
  if (nseg > 1) {
    const dim3 pgrid{unsigned((threads + kComposeThreads - 1) / kComposeThreads), unsigned(nseg), 1u};
    if (vec)
      compose_partial_kernel<DTYPE, true, true><<<pgrid, kComposeThreads, 0, st>>>(a, b, n, S, seg_len, part_a,
                                                                                 part_b, a_stride, b_stride);
    else
      compose_partial_kernel<DTYPE, false, true><<<pgrid, kComposeThreads, 0, st>>>(a, b, n, S, seg_len, part_a,
                                                                                  part_b, a_stride, b_stride);
    CB2_LAUNCH_CHECK();
  }
  const dim3 grid{unsigned(blocks), unsigned(nseg), 1u};
  if (vec)
    prefix_maps_kernel<DTYPE, true, STATES><<<grid, 128, 0, st>>>(a, b, pa, pb, n, S, a_stride, b_stride, seg_len,
                                                                  part_a, part_b, h0);
  else
    prefix_maps_kernel<DTYPE, false, STATES><<<grid, 128, 0, st>>>(a, b, pa, pb, n, S, a_stride, b_stride,
                                                                   seg_len, part_a, part_b, h0);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

int pick_segments(long long n, long long S, int elems_per_thread) {
  long long ctas = (S / elems_per_thread + kComposeThreads - 1) / kComposeThreads;
  if (ctas < 1) ctas = 1;
  long long want = (4 * 148) / ctas;                     // at most one wave of four CTAs per SM
  const long long most = n / 64 > 0 ? n / 64 : 1;        // segments of at least 64 leaves
  if (want > most) want = most;
  if (want < 1) want = 1;
  if (want > 65535) want = 65535;
  return int(want);
}

template <int DTYPE>
int run(const void* a, const void* b, const void* h, void* out, long long n, long long S, void* scratch,
        size_t scratch_bytes, cudaStream_t st, bool chrono = false, long long a_stride = -1,
        long long b_stride = -1) {
  if (a_stride < 0) a_stride = S;
  if (b_stride < 0) b_stride = S;
  using V = Vec<DTYPE>;
  const bool vec = S % V::kElems == 0 && aligned16(a) && aligned16(b);
  const int E = vec ? V::kElems : 1;
  const int nseg = pick_segments(n, S, E);
  const size_t need = size_t(2) * nseg * size_t(S) * sizeof(float);
  if (!scratch || scratch_bytes < need) return CB2_SCRATCH_TOO_SMALL;
  float* part_a = static_cast<float*>(scratch);
  float* part_b = part_a + size_t(nseg) * size_t(S);
  const long long seg_len = (n + nseg - 1) / nseg;
  const long long threads = (S + E - 1) / E;
  const dim3 grid(unsigned((threads + kComposeThreads - 1) / kComposeThreads), unsigned(nseg));
#define CB2_COMPOSE_LAUNCH(VEC_, CHRONO_)                                                        \
  compose_partial_kernel<DTYPE, VEC_, CHRONO_><<<grid, kComposeThreads, 0, st>>>(a, b, n, S, seg_len, \
                                                                                part_a, part_b, a_stride, b_stride)
  if (vec && chrono) CB2_COMPOSE_LAUNCH(true, true);
  else if (vec) CB2_COMPOSE_LAUNCH(true, false);
  else if (chrono) CB2_COMPOSE_LAUNCH(false, true);
  else CB2_COMPOSE_LAUNCH(false, false);
#undef CB2_COMPOSE_LAUNCH
  CB2_LAUNCH_CHECK();
  compose_apply_kernel<DTYPE><<<unsigned((S + kComposeThreads - 1) / kComposeThreads), kComposeThreads, 0, st>>>(
      part_a, part_b, h, out, nseg, S, chrono ? 1 : 0);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace
}  // namespace cb2

extern "C" size_t cb2_diag_compose_scratch_bytes(long long n, long long S, int dtype) {
  if (n <= 0 || S <= 0) return 0;
  // enough for either layout: the 16-byte-vector one has fewer threads per segment
  // and therefore cuts n into more segments
  const int ve = dtype == CB2_BF16 ? 8 : 4;
  const int a = cb2::pick_segments(n, S, 1), b = cb2::pick_segments(n, S, ve);
  return size_t(2) * (a > b ? a : b) * size_t(S) * sizeof(float);
}

extern "C" int cb2_diag_compose_apply(const void* a_seq, const void* b_seq, const void* h, void* out,
                                      long long n, long long S, int dtype, void* scratch,
                                      size_t scratch_bytes, void* stream) {
  if (!a_seq || !b_seq || !h || !out) return CB2_NULL_PTR;
  if (n <= 0 || S <= 0 || S > (1ll << 40) / n) return CB2_BAD_SHAPE;
  if ((S + cb2::kComposeThreads - 1) / cb2::kComposeThreads > 0x7fffffffll) return CB2_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_F32) return cb2::run<CB2_F32>(a_seq, b_seq, h, out, n, S, scratch, scratch_bytes, st);
  if (dtype == CB2_BF16) return cb2::run<CB2_BF16>(a_seq, b_seq, h, out, n, S, scratch, scratch_bytes, st);
  return CB2_UNSUPPORTED_DTYPE;
}

// The same fold for rows stored in TIME order (row 0 = first step):
//     out = f_{n-1}( ... f_1( f_0(h) ) ),   f_j(h) = a_rows[j]*h + b_rows[j],
// the sequence form `applyd(aff_diag(a, b), h)` folded along the step axis that the
// reference's generated scan kernels compute (`_seq_triton_source` / `_seq_binding`,
// catopt_discovery/genkernel.py:1031-1060, 1208-1233).  a_step_stride / b_step_stride:
// elements between consecutive rows, S for one row per step or 0 for a row every step
// shares (a decay that does not depend on the step).
extern "C" int cb2_diag_fold_apply(const void* a_rows, const void* b_rows, const void* h, void* out,
                                   long long n, long long S, long long a_step_stride,
                                   long long b_step_stride, int dtype, void* scratch, size_t scratch_bytes,
                                   void* stream) {
  if (!a_rows || !b_rows || !h || !out) return CB2_NULL_PTR;
  if (n <= 0 || S <= 0 || S > (1ll << 40) / n) return CB2_BAD_SHAPE;
  if ((S + cb2::kComposeThreads - 1) / cb2::kComposeThreads > 0x7fffffffll) return CB2_BAD_SHAPE;
  if ((a_step_stride != 0 && a_step_stride != S) || (b_step_stride != 0 && b_step_stride != S))
    return CB2_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_F32)
    return cb2::run<CB2_F32>(a_rows, b_rows, h, out, n, S, scratch, scratch_bytes, st, true, a_step_stride,
                             b_step_stride);
  if (dtype == CB2_BF16)
    return cb2::run<CB2_BF16>(a_rows, b_rows, h, out, n, S, scratch, scratch_bytes, st, true, a_step_stride,
                              b_step_stride);
  return CB2_UNSUPPORTED_DTYPE;
}

// All prefix maps (Pa[t], Pb[t]) of rows in time order, h_t = Pa[t]*h_0 + Pb[t]: what
// `BatchedOmdModule._prefix_scan` (catopt_carriers/omd_lower.py:771-824) builds from blocks of
// sqrt(T) serial compose steps plus a carry fold; here one pass that reads a and b once and
// writes both maps once.  a_rows, b_rows: [n, S] (step stride S, or 0 for a shared row);
// pa, pb: [n, S], element type `dtype`; fp32 running maps.  With scratch
// (cb2_diag_prefix_maps_scratch_bytes) a state too small to fill the GPU is made up for by cutting
// the steps into segments (totals first, then every segment from its carry-in).
extern "C" size_t cb2_diag_prefix_maps_scratch_bytes(long long n, long long S, int dtype) {
  if (n <= 0 || S <= 0) return 0;
  const int ve = dtype == CB2_BF16 ? 8 : 4;
  const int a = cb2::prefix_segments(n, S, 1), b = cb2::prefix_segments(n, S, ve);
  const int m = a > b ? a : b;
  return m > 1 ? size_t(2) * m * size_t(S) * sizeof(float) : 0;
}

extern "C" int cb2_diag_prefix_maps(const void* a_rows, const void* b_rows, void* pa, void* pb, long long n,
                                    long long S, long long a_step_stride, long long b_step_stride,
                                    int dtype, void* scratch, size_t scratch_bytes, void* stream) {
  if (!a_rows || !b_rows || !pa || !pb) return CB2_NULL_PTR;
  if (n <= 0 || S <= 0 || S > (1ll << 40) / n) return CB2_BAD_SHAPE;
  if ((a_step_stride != 0 && a_step_stride != S) || (b_step_stride != 0 && b_step_stride != S))
    return CB2_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_F32)
    return cb2::run_prefix<CB2_F32>(a_rows, b_rows, pa, pb, n, S, a_step_stride, b_step_stride, scratch,
                                    scratch_bytes, st);
  if (dtype == CB2_BF16)
    return cb2::run_prefix<CB2_BF16>(a_rows, b_rows, pa, pb, n, S, a_step_stride, b_step_stride, scratch,
                                     scratch_bytes, st);
  return CB2_UNSUPPORTED_DTYPE;
}

// Every state of a diagonal recurrence over time-ordered step rows: out[t] = a_t*out[t-1] + b_t with
// out[-1] = h — the value of `applyd(aff_diag(stack(affd_a f_t), stack(affd_b f_t)), h)` over the
// prefix maps f_t = leaf_t . f_(t-1), the stacked-map form `gather_applyd_stack` offers for an
// unrolled scan (catopt_carriers/xcarrier.py:2252-2275), which the reference evaluates one compose
// per step.  One pass: a and b read once, the states written once (fp32 running state); segments
// through scratch as in cb2_diag_prefix_maps (same scratch query).
extern "C" int cb2_diag_scan_states(const void* a_rows, const void* b_rows, const void* h, void* out, long long n,
                                    long long S, long long a_step_stride, long long b_step_stride, int dtype,
                                    void* scratch, size_t scratch_bytes, void* stream) {
  if (!a_rows || !b_rows || !h || !out) return CB2_NULL_PTR;
  if (n <= 0 || S <= 0 || S > (1ll << 40) / n) return CB2_BAD_SHAPE;
  if ((a_step_stride != 0 && a_step_stride != S) || (b_step_stride != 0 && b_step_stride != S))
    return CB2_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_F32)
    return cb2::run_prefix<CB2_F32, true>(a_rows, b_rows, nullptr, out, n, S, a_step_stride, b_step_stride, scratch,
                                          scratch_bytes, st, h);
  if (dtype == CB2_BF16)
    return cb2::run_prefix<CB2_BF16, true>(a_rows, b_rows, nullptr, out, n, S, a_step_stride, b_step_stride,
                                           scratch, scratch_bytes, st, h);
  return CB2_UNSUPPORTED_DTYPE;
}
