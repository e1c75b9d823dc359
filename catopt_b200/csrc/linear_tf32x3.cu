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
// w is split once per call by a small kernel into caller-provided scratch, so
// its hi/lo tiles arrive by TMA ready to use as the shared-memory (B) operand.
// Persistent CTAs (one per SM) walk 128 x 128 output tiles.  Roles: warp 0
// streams 128 x 32 fp32 tiles of x, w_hi and w_lo through a 4-stage ring with TMA
// (128-byte swizzle, K-major: x and nn.Linear weights are row-major over the
// reduction axis); warps 2..5 read each x tile once (thread = row), split it in
// registers and park hi and lo in TENSOR MEMORY, from where the MMAs take them
// as the A operand — an SS-form tf32 MMA reads 128 B/clk of shared memory, all
// the port has, so keeping x out of shared memory is what lets the three passes
// run near the tensor rate; warp 1 issues the MMAs into one of two TMEM
// accumulators and releases stages with tcgen05.commit; warps 6..9 drain the
// other accumulator (bias, store rows of y) while the next tile is being
// multiplied.  Out-of-range rows/columns are zero-filled by the TMA.
// Measured at R = 65536, 512 -> 512: the tensor pipe is active 73 % of the
// cycles (three tf32 passes = 103 GFLOP); each CTA pulls 48 KB per 32-deep step
// from L2 (x + w_hi + w_lo tiles, 1.6 GB per call, a third of the L2 -> SM peak).
// TMEM map (512 columns): accumulators at 0 and 128; x slot s at 256 + 64 s
// (hi 32 columns, lo 32 columns).
#include <algorithm>

#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kStages = 4;
constexpr int kThreads = 320;                          // TMA, MMA, 4 split warps, 4 epilogue warps
constexpr uint32_t kTileB = 128 * 128;                 // 128 rows x 32 fp32 = 16 KiB
constexpr uint32_t kStageB = 3 * kTileB;               // x | w_hi | w_lo
constexpr uint32_t kOffBars = kStages * kStageB;
constexpr int kNumBars = 3 * kStages + 4;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColX = 256;                        // x slots: 64 columns per stage
// The tensor-core accumulator adds with truncation, which shrinks a sum by a factor that grows with
// the number of additions (measured rel-err 3e-6 at 512 products per output, 5e-6 at 1024, 1.1e-5 at
// 2048).  A tensor-memory accumulator therefore takes at most kSegBlocks 32-deep k-blocks; a deeper
// reduction is cut into segments of half that (512 products) whose sums the epilogue adds in fp32
// (the first segment stores y, the others add to it), which keeps the error at the 512-deep level
// whatever the depth.
constexpr int kSegBlocks = 32;

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

__global__ void w_split_kernel(const float4* __restrict__ w, float4* __restrict__ hi, float4* __restrict__ lo,
                               size_t n4) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n4; i += size_t(gridDim.x) * blockDim.x) {
    const float4 v = w[i];
    float4 h, l;
    h.x = tf32_rn(v.x); l.x = v.x - h.x;
    h.y = tf32_rn(v.y); l.y = v.y - h.y;
    h.z = tf32_rn(v.z); l.z = v.z - h.z;
    h.w = tf32_rn(v.w); l.w = v.w - h.w;
    hi[i] = h;
    lo[i] = l;
  }
}

// A operand from tensor memory (lane = row, one tf32 per column), B from shared memory.
__device__ __forceinline__ void mma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
linear_tf32x3_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_whi,
                     const __grid_constant__ CUtensorMap map_wlo, const float* __restrict__ bias,
                     float* __restrict__ y, int R, int n_in, int n_out, int tiles_n, int n_tiles,
                     int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* full = bars;                      // TMA -> splitters
  uint64_t* split = bars + kStages;           // splitters -> MMA (128 arrivals)
  uint64_t* empty = bars + 2 * kStages;       // MMA -> TMA
  uint64_t* acc_full = bars + 3 * kStages;    // MMA -> epilogue   [2]
  uint64_t* acc_empty = acc_full + 2;         // epilogue -> MMA   [2] (128 arrivals)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nkb = (n_in + 31) / 32;
  const int seg = nkb <= kSegBlocks ? kSegBlocks : kSegBlocks / 2;   // k-blocks per accumulator

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&split[s], 128);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
    }
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    umma::tmem_alloc(s_tmem, kTmemCols);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  if (warp == 0) {
    if (lane == 0) {
      umma::tma_prefetch_desc(&map_x);
      umma::tma_prefetch_desc(&map_whi);
      umma::tma_prefetch_desc(&map_wlo);
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * 128, n0 = (tile % tiles_n) * 128;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % kStages, use = it / kStages;
          if (use > 0 && !mbar_wait_abortable(&empty[s], (use - 1) & 1, s_abort)) { ok = false; break; }
          unsigned char* st = smem + s * kStageB;
          mbar_arrive_expect_tx(&full[s], 3 * kTileB);
          umma::tma_load_2d(st, &map_x, kb * 32, m0, &full[s]);
          umma::tma_load_2d(st + kTileB, &map_whi, kb * 32, n0, &full[s]);
          umma::tma_load_2d(st + 2 * kTileB, &map_wlo, kb * 32, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_tf32(128, 128);
      int it = 0, tl = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
        for (int kb0 = 0; ok && kb0 < nkb; kb0 += seg, ++tl) {
          const int buf = tl & 1, use = tl >> 1;
          if (use > 0 && !mbar_wait_abortable(&acc_empty[buf], (use - 1) & 1, s_abort)) { ok = false; break; }
          umma::fence_after_sync();
          const uint32_t acc = tmem + buf * 128u;
          const int kb1 = min(nkb, kb0 + seg);
          for (int kb = kb0; kb < kb1; ++kb, ++it) {
            const int s = it % kStages;
            if (!mbar_wait_abortable(&split[s], (it / kStages) & 1, s_abort)) { ok = false; break; }
            umma::fence_after_sync();
            const uint32_t wbase = smem_u32(smem + s * kStageB + kTileB);
            const uint32_t xh = tmem + kColX + s * 64u, xl = xh + 32u;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const uint64_t wh = umma::smem_desc(wbase + ks * 32u, 16u, 1024u);
              const uint64_t wl = umma::smem_desc(wbase + kTileB + ks * 32u, 16u, 1024u);
              mma_tf32_ts(acc, xl + ks * 8u, wh, idesc, (kb > kb0) || (ks > 0));   // small terms first
              mma_tf32_ts(acc, xh + ks * 8u, wl, idesc, true);
              mma_tf32_ts(acc, xh + ks * 8u, wh, idesc, true);
            }
            umma::mma_commit(&empty[s]);
          }
          if (ok) umma::mma_commit(&acc_full[buf]);
        }
      }
    }
  } else if (warp < 6) {
    // splitters: thread = one row; warp w owns TMEM lanes 32*(w % 4)..+31
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const uint32_t lane_base = tmem + kColX + (uint32_t(q4 * 32) << 16);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % kStages;
        ok = mbar_wait_abortable(&full[s], (it / kStages) & 1, s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const unsigned char* xrow = smem + s * kStageB + r * 128u;
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // logical 16-byte chunk j of row r sits at physical chunk j ^ (r % 8) (128-byte
          // swizzle); a quarter-warp thereby touches eight different bank groups
          const float4 v = *reinterpret_cast<const float4*>(xrow + uint32_t((j ^ (r & 7)) * 16));
          const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float h = tf32_rn(e[t]);
            hi[4 * j + t] = __float_as_uint(h);
            lo[4 * j + t] = __float_as_uint(e[t] - h);
          }
        }
        umma::tmem_st32(lane_base + s * 64u, hi);
        umma::tmem_st32(lane_base + s * 64u + 32u, lo);
        umma::tmem_wait_st();
        umma::fence_before_sync();
        mbar_arrive(&split[s]);
      }
    }
  } else {
    // epilogue: warp w reads TMEM lanes 32*(w % 4)..+31 = rows of the tile
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    int tl = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      const int m0 = (tile / tiles_n) * 128, n0 = (tile % tiles_n) * 128;
      const int gm = m0 + r;
      for (int kb0 = 0; kb0 < nkb; kb0 += seg, ++tl) {
        const int buf = tl & 1;
        ok = mbar_wait_abortable(&acc_full[buf], (tl >> 1) & 1, s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        umma::fence_after_sync();
        // the first segment of a tile stores y (+ bias); later ones add to what this same
        // thread stored before
        const bool add = kb0 > 0;
        const uint32_t lane_base = tmem + buf * 128u + (uint32_t(q4 * 32) << 16);
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
                if (add) {
                  const float4 p = *reinterpret_cast<const float4*>(yrow + j);
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                } else if (bias) {
                  const float4 bb = *reinterpret_cast<const float4*>(bias + gn);
                  o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                }
                *reinterpret_cast<float4*>(yrow + j) = o;
              } else {
                const float oo[4] = {o.x, o.y, o.z, o.w};
                for (int t = 0; t < 4; ++t)
                  if (gn + t < n_out) yrow[j + t] = oo[t] + (add ? yrow[j + t] : (bias ? bias[gn + t] : 0.f));
              }
            }
          }
        }
        umma::fence_before_sync();
        mbar_arrive(&acc_empty[buf]);
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
    umma::tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

// Used by cb2_linear_f32: large row counts with TMA-compatible strides, and
// scratch for the split weight (without it the call stays on the FMA pipes).
bool linear_tf32x3_supported(const float* x, const float* w, const float* bias, const float* y, int R,
                             int n_in, int n_out, const void* scratch, size_t scratch_bytes) {
  // any reduction depth: deep ones are cut into accumulator segments (kSegBlocks)
  return R >= 256 && n_in % 4 == 0 && n_out % 4 == 0 && aligned16(x) && aligned16(w) &&
         aligned16(y) && (!bias || aligned16(bias)) && scratch && aligned16(scratch) &&
         scratch_bytes >= size_t(2) * n_in * n_out * sizeof(float);
}

// Bytes of scratch for the split weight (hi then lo, each [out, in] fp32).
size_t linear_tf32x3_scratch_bytes(int n_in, int n_out) { return size_t(2) * n_in * n_out * sizeof(float); }

// w -> TF32 hi part and exact remainder, [out, in] fp32 each, hi then lo in `w_split`.
int linear_tf32x3_split(const float* w, float* w_split, int n_in, int n_out, cudaStream_t st) {
  const size_t wn = size_t(n_in) * n_out;
  const size_t n4 = wn / 4;   // n_in % 4 == 0
  w_split_kernel<<<unsigned(std::min<size_t>((n4 + 255) / 256, 592)), 256, 0, st>>>(
      reinterpret_cast<const float4*>(w), reinterpret_cast<float4*>(w_split),
      reinterpret_cast<float4*>(w_split + wn), n4);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

// The GEMM on an already split weight (a module whose weight never changes splits it once).
int linear_tf32x3_run_presplit(const float* x, const float* w_split, const float* bias, float* y, int R, int n_in,
                               int n_out, int* dev_status, cudaStream_t st) {
  const size_t wn = size_t(n_in) * n_out;
  const float* w_hi = w_split;
  const float* w_lo = w_hi + wn;
  CUtensorMap mx, mwhi, mwlo;
  int rc = make_f32_map(&mx, x, R, n_in);
  if (rc == CB2_OK) rc = make_f32_map(&mwhi, w_hi, n_out, n_in);
  if (rc == CB2_OK) rc = make_f32_map(&mwlo, w_lo, n_out, n_in);
  if (rc != CB2_OK) return rc;
  if (cudaFuncSetAttribute(linear_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           int(kSmemBytes)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  const int tiles_n = (n_out + 127) / 128, tiles_m = (R + 127) / 128;
  const long long n_tiles = (long long)tiles_n * tiles_m;
  if (n_tiles > 0x7fffffffLL) return CB2_BAD_SHAPE;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned grid = unsigned(std::min<long long>(n_tiles, sms));
  linear_tf32x3_kernel<<<grid, kThreads, kSmemBytes, st>>>(mx, mwhi, mwlo, bias, y, R, n_in, n_out, tiles_n,
                                                           int(n_tiles), dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

int linear_tf32x3_run(const float* x, const float* w, const float* bias, float* y, int R, int n_in,
                      int n_out, void* scratch, int* dev_status, cudaStream_t st) {
  float* w_split = static_cast<float*>(scratch);
  const int rc = linear_tf32x3_split(w, w_split, n_in, n_out, st);
  if (rc != CB2_OK) return rc;
  return linear_tf32x3_run_presplit(x, w_split, bias, y, R, n_in, n_out, dev_status, st);
}

}  // namespace cb2
