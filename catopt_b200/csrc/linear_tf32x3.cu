// y[R,out] = x[R,in] . w[out,in]^T (+ bias) in fp32 on the tensor cores with
// three-pass TF32 splitting, for the runtime GEMM of a folded weight chain
// (`linear(input, fused_N)`, catopt_torch/torch_bridge.py:1251-1253) when the
// batch of rows is large enough to fill 128-row tiles.
//
// A single TF32 pass keeps 10 mantissa bits (rel-err ~5e-4), far from the 1e-5
// this path promises.  Each fp32 operand is therefore split on the fly into
//   hi = the operand rounded to the nearest TF32 value (10 mantissa bits)
//   lo = operand - hi                                     (exact in fp32, <= 2^-11 |operand|)
// and the product is accumulated in fp32 tensor memory as
//   hi.hi + hi.lo + lo.hi            (the dropped lo.lo term is ~2^-22 relative),
// three tcgen05.mma kind::tf32 per 8-deep step.
//
// CTA = one 128 x 128 output tile.  Roles: warp 0 streams 128 x 32 fp32 tiles of
// x and w through a 3-stage ring with TMA (128-byte swizzle, K-major for both
// operands since x and nn.Linear weights are row-major over the reduction
// axis); warps 2..5 split each stage in shared memory (hi in place, lo into a
// second buffer); warp 1 issues the MMAs and releases stages with
// tcgen05.commit; warps 2..5 finally read the accumulator, add the bias and
// store rows of y.  Out-of-range rows/columns are zero-filled by the TMA.
#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kStages = 3;
constexpr int kThreads = 192;
constexpr uint32_t kTileB = 128 * 128;                 // 128 rows x 32 fp32 = 16 KiB
constexpr uint32_t kStageB = 4 * kTileB;               // x_hi | x_lo | w_hi | w_lo
constexpr uint32_t kOffBars = kStages * kStageB;
constexpr int kNumBars = 3 * kStages + 1;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;

__host__ __device__ constexpr uint32_t instr_desc_tf32(uint32_t M, uint32_t N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}

// Nearest TF32 value (10 explicit mantissa bits): the residual v - tf32_rn(v) is
// exact in fp32 and at most 2^-11 |v|.
__device__ __forceinline__ float tf32_rn(float v) {
  return __uint_as_float((__float_as_uint(v) + 0x1000u) & 0xffffe000u);
}

// fp32 row-major [rows x cols] matrix, box {32 columns, 128 rows}, 128-byte swizzle.
int make_f32_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols) {
  using Fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                          const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                          CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !p)
      return CB2_LAUNCH_FAIL;
    fn = reinterpret_cast<Fn>(p);
  }
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {cols * 4};
  const cuuint32_t box[2] = {32, 128};
  const cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? CB2_OK
             : CB2_LAUNCH_FAIL;
}

__global__ void __launch_bounds__(kThreads, 1)
linear_tf32x3_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     const float* __restrict__ bias, float* __restrict__ y, int R, int n_in, int n_out,
                     int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* full = bars;                    // TMA -> splitters
  uint64_t* split = bars + kStages;         // splitters -> MMA (128 arrivals)
  uint64_t* empty = bars + 2 * kStages;     // MMA -> TMA
  uint64_t* acc_ready = bars + 3 * kStages; // MMA -> epilogue
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * 128, n0 = blockIdx.x * 128;
  const int nkb = (n_in + 31) / 32;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&split[s], 128);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    umma::tmem_alloc(s_tmem, 128);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  if (warp == 0) {
    if (lane == 0) {
      umma::tma_prefetch_desc(&map_x);
      umma::tma_prefetch_desc(&map_w);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % kStages, use = kb / kStages;
        if (use > 0 && !mbar_wait_abortable(&empty[s], (use - 1) & 1, s_abort)) break;
        unsigned char* st = smem + s * kStageB;
        mbar_arrive_expect_tx(&full[s], 2 * kTileB);
        umma::tma_load_2d(st, &map_x, kb * 32, m0, &full[s]);               // raw x -> x_hi slot
        umma::tma_load_2d(st + 2 * kTileB, &map_w, kb * 32, n0, &full[s]);  // raw w -> w_hi slot
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_tf32(128, 128);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % kStages;
        if (!mbar_wait_abortable(&split[s], (kb / kStages) & 1, s_abort)) break;
        umma::fence_after_sync();
        const uint32_t base = smem_u32(smem + s * kStageB);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t xh = umma::smem_desc(base + ks * 32u, 16u, 1024u);
          const uint64_t xl = umma::smem_desc(base + kTileB + ks * 32u, 16u, 1024u);
          const uint64_t wh = umma::smem_desc(base + 2 * kTileB + ks * 32u, 16u, 1024u);
          const uint64_t wl = umma::smem_desc(base + 3 * kTileB + ks * 32u, 16u, 1024u);
          mma_tf32(tmem, xl, wh, idesc, (kb > 0) || (ks > 0));   // small terms first
          mma_tf32(tmem, xh, wl, idesc, true);
          mma_tf32(tmem, xh, wh, idesc, true);
        }
        umma::mma_commit(&empty[s]);
      }
      umma::mma_commit(acc_ready);
    }
  } else {
    // splitters / epilogue: thread = one row of the 128-row tiles
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % kStages;
      bool ok = mbar_wait_abortable(&full[s], (kb / kStages) & 1, s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      unsigned char* st = smem + s * kStageB;
#pragma unroll
      for (int op = 0; op < 2; ++op) {      // 0: x, 1: w
        unsigned char* hi_t = st + op * 2 * kTileB;
        unsigned char* lo_t = hi_t + kTileB;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // The 128-byte swizzle only permutes the 16-byte chunks inside a row and the
          // same permutation applies to the hi and the lo tile, so the split can walk
          // physical chunks; starting each lane at chunk (r % 8) keeps a quarter-warp
          // on eight different bank groups.
          const uint32_t off = r * 128u + uint32_t((j ^ (r & 7)) * 16);
          float4 v = *reinterpret_cast<const float4*>(hi_t + off);
          float4 h, l;
          h.x = tf32_rn(v.x); l.x = v.x - h.x;
          h.y = tf32_rn(v.y); l.y = v.y - h.y;
          h.z = tf32_rn(v.z); l.z = v.z - h.z;
          h.w = tf32_rn(v.w); l.w = v.w - h.w;
          *reinterpret_cast<float4*>(hi_t + off) = h;
          *reinterpret_cast<float4*>(lo_t + off) = l;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&split[s]);
    }
    bool ok = mbar_wait_abortable(acc_ready, 0, s_abort);
    if (__all_sync(0xffffffffu, ok)) {
      umma::fence_after_sync();
      const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
      const int gm = m0 + r;
      uint32_t v[32];
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        umma::tmem_ld32(lane_base + cb * 32, v);
        umma::tmem_wait_ld();
        if (gm < R) {
          float* yrow = y + size_t(gm) * n_out + n0 + cb * 32;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int gn = n0 + cb * 32 + j;
            float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                   __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            if (gn + 3 < n_out) {
              if (bias) {
                const float4 bb = *reinterpret_cast<const float4*>(bias + gn);
                o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
              }
              *reinterpret_cast<float4*>(yrow + j) = o;
            } else {
              const float oo[4] = {o.x, o.y, o.z, o.w};
              for (int t = 0; t < 4; ++t)
                if (gn + t < n_out) yrow[j + t] = oo[t] + (bias ? bias[gn + t] : 0.f);
            }
          }
        }
      }
    }
  }
  __syncwarp();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  if (tid == 0 && *s_abort && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT);
  if (warp == 1) {
    __syncwarp();
    umma::tmem_dealloc(tmem, 128);
  }
}

}  // namespace

// Used by cb2_linear_f32: large row counts with TMA-compatible strides.
bool linear_tf32x3_supported(const float* x, const float* w, const float* bias, const float* y, int R,
                             int n_in, int n_out) {
  // The tensor-core accumulator adds with truncation, a bias that grows with the
  // reduction depth: measured rel-err 3e-6 at in=512, 5e-6 at 1024, 1.1e-5 at
  // 2048.  Deeper reductions stay on the FMA pipes to keep the 1e-5 promise.
  return R >= 256 && n_in <= 1024 && n_in % 4 == 0 && n_out % 4 == 0 && aligned16(x) && aligned16(w) &&
         aligned16(y) && (!bias || aligned16(bias));
}

int linear_tf32x3_run(const float* x, const float* w, const float* bias, float* y, int R, int n_in,
                      int n_out, int* dev_status, cudaStream_t st) {
  CUtensorMap mx, mw;
  int rc = make_f32_map(&mx, x, R, n_in);
  if (rc == CB2_OK) rc = make_f32_map(&mw, w, n_out, n_in);
  if (rc != CB2_OK) return rc;
  if (cudaFuncSetAttribute(linear_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           int(kSmemBytes)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  dim3 grid((n_out + 127) / 128, (R + 127) / 128);
  linear_tf32x3_kernel<<<grid, kThreads, kSmemBytes, st>>>(mx, mw, bias, y, R, n_in, n_out, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
