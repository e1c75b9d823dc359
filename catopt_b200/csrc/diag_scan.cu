// Diagonal linear recurrence with readout,
//   h_t[n] = a_t[n] * h_{t-1}[n] + b[n] * x_t,   y_t = sum_n c[n] * h_t[n],
// one step of which is the reference's applyd(aff_diag(a_t, b*x_t), h)
// (catopt_torch/torch_bridge.py:1895-1900).
//
// Bandwidth kernel: `a` ([B,T,D,N]) is read exactly once and dominates the
// traffic (algorithmic bytes per (b,t) position = D*(N+2)*sizeof(elem)).
//
// Layout / mapping.  A CTA owns one batch entry and a block of kCh channels
// for the whole sequence; a thread owns kNpt consecutive n of one channel
// (16 bytes of bf16), its states live in registers for all T steps, and the
// n-sum of the readout finishes with warp shuffles across the kLpc lanes that
// share a channel.  The T axis is streamed through a kStages-deep ring of
// shared-memory tiles of kRows time steps, filled by the TMA engine with one
// bulk copy per row (a row of the block is kCh*N contiguous elements) and
// tracked by one mbarrier per stage, so kStages-1 tiles per CTA are always in
// flight while the serial recurrence runs on the resident one.  y is staged in
// shared memory and written with 16-byte stores.
#include <cstdlib>
#include <type_traits>

#include "umma.cuh"

namespace cb2 {
namespace {

template <int DTYPE>
struct Elem;
template <>
struct Elem<CB2_BF16> {
  using T = __nv_bfloat16;
  static constexpr int kSize = 2;
  __device__ static float ld(const void* p, int i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
  __device__ static void st(void* p, int i, float v) {
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  }
};
template <>
struct Elem<CB2_F32> {
  using T = float;
  static constexpr int kSize = 4;
  __device__ static float ld(const void* p, int i) { return static_cast<const float*>(p)[i]; }
  __device__ static void st(void* p, int i, float v) { static_cast<float*>(p)[i] = v; }
};

template <int DTYPE, int N>
struct ScanCfg {
  static constexpr int kEsz = Elem<DTYPE>::kSize;
  static constexpr int kNpt = N < 8 ? N : 8;          // n per thread
  static constexpr int kLpc = N / kNpt;               // lanes per channel
  static constexpr int kThreads = 64;
  static constexpr int kCh = kThreads / kLpc;         // channels per CTA
  static constexpr int kRows = DTYPE == CB2_BF16 ? 16 : 8;  // time steps per tile
  static constexpr int kStages = 4;
  static constexpr int kARow = kCh * N * kEsz;        // bytes of `a` per time step
  static constexpr int kXRow = kCh * kEsz;            // bytes of x (and y) per time step
  static constexpr int kStageBytes = kRows * (kARow + kXRow);
  static constexpr int kYBytes = kRows * kXRow;
  static constexpr int kSmem = kStages * kStageBytes + 2 * kYBytes + kStages * 8 + 16;
};

// Widen kNpt consecutive elements starting at byte pointer p into f[].
template <int DTYPE, int NPT>
__device__ __forceinline__ void load_row(const unsigned char* p, float (&f)[NPT]) {
  if constexpr (DTYPE == CB2_BF16) {
    if constexpr (NPT == 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(p);
      f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x);
      f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
      f[4] = bf16lo_to_f32(v.z); f[5] = bf16hi_to_f32(v.z);
      f[6] = bf16lo_to_f32(v.w); f[7] = bf16hi_to_f32(v.w);
    } else if constexpr (NPT == 4) {
      const uint2 v = *reinterpret_cast<const uint2*>(p);
      f[0] = bf16lo_to_f32(v.x); f[1] = bf16hi_to_f32(v.x);
      f[2] = bf16lo_to_f32(v.y); f[3] = bf16hi_to_f32(v.y);
    } else if constexpr (NPT == 2) {
      const uint32_t v = *reinterpret_cast<const uint32_t*>(p);
      f[0] = bf16lo_to_f32(v); f[1] = bf16hi_to_f32(v);
    } else {
      f[0] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
    }
  } else {
    if constexpr (NPT == 8) {
      const float4 v0 = *reinterpret_cast<const float4*>(p);
      const float4 v1 = *reinterpret_cast<const float4*>(p + 16);
      f[0] = v0.x; f[1] = v0.y; f[2] = v0.z; f[3] = v0.w;
      f[4] = v1.x; f[5] = v1.y; f[6] = v1.z; f[7] = v1.w;
    } else if constexpr (NPT == 4) {
      const float4 v0 = *reinterpret_cast<const float4*>(p);
      f[0] = v0.x; f[1] = v0.y; f[2] = v0.z; f[3] = v0.w;
    } else if constexpr (NPT == 2) {
      const float2 v0 = *reinterpret_cast<const float2*>(p);
      f[0] = v0.x; f[1] = v0.y;
    } else {
      f[0] = *reinterpret_cast<const float*>(p);
    }
  }
}

template <int DTYPE, int N>
__global__ void __launch_bounds__(64)
diag_scan_kernel(const unsigned char* __restrict__ a, const unsigned char* __restrict__ x,
                 const void* __restrict__ bvec, const void* __restrict__ cvec,
                 const float* __restrict__ h0, unsigned char* __restrict__ y,
                 float* __restrict__ hT, int T, int D, int* dev_status) {
  using C = ScanCfg<DTYPE, N>;
  using E = Elem<DTYPE>;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_stage = smem;                                   // kStages x [a rows | x rows]
  unsigned char* s_y = smem + C::kStages * C::kStageBytes;         // 2 x kYBytes
  uint64_t* s_full = reinterpret_cast<uint64_t*>(s_y + 2 * C::kYBytes);

  const int tid = threadIdx.x;
  const int blocks_per_b = (D + C::kCh - 1) / C::kCh;
  const int b = blockIdx.x / blocks_per_b;
  const int d0 = (blockIdx.x % blocks_per_b) * C::kCh;
  const int nch = min(C::kCh, D - d0);                             // channels this CTA owns
  const int ch = tid / C::kLpc, sub = tid % C::kLpc;
  const bool live = ch < nch;
  const int d = d0 + ch;
  const uint32_t a_row_bytes = uint32_t(nch) * N * C::kEsz;
  const uint32_t x_row_bytes = uint32_t(nch) * C::kEsz;
  const size_t a_row_stride = size_t(D) * N * C::kEsz;
  const size_t x_row_stride = size_t(D) * C::kEsz;
  const unsigned char* a_base = a + (size_t(b) * T * D + d0) * N * C::kEsz;
  const unsigned char* x_base = x + (size_t(b) * T * D + d0) * C::kEsz;
  unsigned char* y_base = y + (size_t(b) * T * D + d0) * C::kEsz;
  const int ntiles = (T + C::kRows - 1) / C::kRows;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) mbar_init(&s_full[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // Producer: warp 0 fills stage (tile % kStages) with tile's rows.
  auto issue_tile = [&](int tile) {
    const int s = tile % C::kStages;
    const int t0 = tile * C::kRows;
    const int rows = min(C::kRows, T - t0);
    unsigned char* sa = s_stage + s * C::kStageBytes;
    unsigned char* sx = sa + C::kRows * C::kARow;
    if (tid == 0) mbar_arrive_expect_tx(&s_full[s], uint32_t(rows) * (a_row_bytes + x_row_bytes));
    __syncwarp();
    if (tid < rows) {
      bulk_g2s(sa + tid * C::kARow, a_base + size_t(t0 + tid) * a_row_stride, a_row_bytes,
               &s_full[s]);
      bulk_g2s(sx + tid * C::kXRow, x_base + size_t(t0 + tid) * x_row_stride, x_row_bytes,
               &s_full[s]);
    }
  };
  if (tid < 32) {
    for (int i = 0; i < C::kStages && i < ntiles; ++i) issue_tile(i);
  }

  float h[C::kNpt], bw[C::kNpt], cw[C::kNpt];
#pragma unroll
  for (int j = 0; j < C::kNpt; ++j) {
    const int n = sub * C::kNpt + j;
    bw[j] = live ? E::ld(bvec, d * N + n) : 0.f;
    cw[j] = live ? E::ld(cvec, d * N + n) : 0.f;
    h[j] = (live && h0) ? h0[(size_t(b) * D + d) * N + n] : 0.f;
  }

  for (int tile = 0; tile < ntiles; ++tile) {
    const int s = tile % C::kStages;
    const uint32_t parity = (tile / C::kStages) & 1;
    const int t0 = tile * C::kRows;
    const int rows = min(C::kRows, T - t0);
    const bool ok = mbar_wait_bounded(&s_full[s], parity);
    const unsigned char* sa = s_stage + s * C::kStageBytes + tid * (C::kNpt * C::kEsz);
    const unsigned char* sx = s_stage + s * C::kStageBytes + C::kRows * C::kARow + ch * C::kEsz;
    unsigned char* sy = s_y + (tile & 1) * C::kYBytes;
    if (ok) {
#pragma unroll 4
      for (int r = 0; r < C::kRows; ++r) {
        if (r < rows) {
          float av[C::kNpt];
          load_row<DTYPE, C::kNpt>(sa + r * C::kARow, av);
          const float xv = E::ld(sx + r * C::kXRow, 0);
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < C::kNpt; ++j) {
            h[j] = fmaf(av[j], h[j], bw[j] * xv);
            acc = fmaf(cw[j], h[j], acc);
          }
#pragma unroll
          for (int off = C::kLpc >> 1; off > 0; off >>= 1)
            acc += __shfl_xor_sync(0xffffffffu, acc, off);
          if (sub == 0) E::st(sy + r * C::kXRow, ch, acc);
        }
      }
    }
    // Everyone is done with stage s and has written its y rows; a failed wait
    // anywhere in the CTA ends the loop for all of its threads.
    if (__syncthreads_or(!ok)) {
      if (tid == 0 && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT);
      return;
    }
    if (tid < 32 && tile + C::kStages < ntiles) issue_tile(tile + C::kStages);
    // y tile -> global, 16 bytes per thread per pass.
    const int vec_per_row = int(x_row_bytes) / 16;
    for (int i = tid; i < rows * vec_per_row; i += C::kThreads) {
      const int r = i / vec_per_row, piece = i % vec_per_row;
      const uint4 v = *reinterpret_cast<const uint4*>(sy + r * C::kXRow + piece * 16);
      *reinterpret_cast<uint4*>(y_base + size_t(t0 + r) * x_row_stride + piece * 16) = v;
    }
  }

  if (hT && live) {
#pragma unroll
    for (int j = 0; j < C::kNpt; ++j)
      hT[(size_t(b) * D + d) * N + sub * C::kNpt + j] = h[j];
  }
}

// ---------------------------------------------------------------------------
// Fast path (D a multiple of 32, N >= 4): same ownership of channels and
// states, but
//  * tiles come in through tiled TMA (3-D tensor maps {D*N | D, T, B}: a tile of
//    16 time steps is kNumBox + 1 copies instead of 32 row copies, and the T
//    axis is clipped per batch entry by the map itself);
//  * a dedicated producer warp issues every copy and the y stores; consumer
//    warps hand stages back through an `empty` mbarrier and never meet at a
//    CTA-wide barrier, so they drift apart and hide each other's latencies;
//  * a thread owns NPT n (4 lanes per channel for N=16), the arithmetic runs on
//    two-wide fp32 FMAs, operands of the next four steps are loaded while the
//    current four are computed, and the n-sum is a transposing shuffle
//    reduction that leaves each lane with the total of ONE step;
//  * y goes out with one TMA store per tile from a double-buffered staging area.
// ---------------------------------------------------------------------------
template <int DTYPE, int N, int NPT>
struct FastCfg {
  static constexpr int kEsz = Elem<DTYPE>::kSize;
  static constexpr int kNpt = NPT;
  static constexpr int kLpc = N / NPT;
  static constexpr int kCh = 32;
  static constexpr int kConsumers = kCh * kLpc;
  static constexpr int kThreads = kConsumers + 32;     // + producer warp
  static constexpr int kRows = 16;
  static constexpr int kStages = 4;
  static constexpr int kRowElems = kCh * N;
  static constexpr int kBoxCols = kRowElems < 256 ? kRowElems : 256;
  static constexpr int kNumBox = kRowElems / kBoxCols;
  static constexpr int kABytes = kRows * kRowElems * kEsz;
  static constexpr int kXBytes = kRows * kCh * kEsz;
  static constexpr int kStageBytes = kABytes + kXBytes;
  static constexpr int kNumBars = 2 * kStages + 2;
  static constexpr int kSmem = kStages * kStageBytes + 2 * kXBytes + kNumBars * 8 + 16 + 128;
};

template <int DTYPE, int N, int NPT>
__global__ void __launch_bounds__(FastCfg<DTYPE, N, NPT>::kThreads)
diag_scan_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_x,
                     const __grid_constant__ CUtensorMap map_y, const void* __restrict__ bvec,
                     const void* __restrict__ cvec, const float* __restrict__ h0,
                     float* __restrict__ hT, int T, int D, int* dev_status) {
  using C = FastCfg<DTYPE, N, NPT>;
  using E = Elem<DTYPE>;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_stage = smem;
  unsigned char* s_y = smem + C::kStages * C::kStageBytes;
  uint64_t* s_full = reinterpret_cast<uint64_t*>(s_y + 2 * C::kXBytes);   // [kStages] TMA -> consumers
  uint64_t* s_empty = s_full + C::kStages;                                // [kStages] consumers -> producer
  uint64_t* s_yfree = s_empty + C::kStages;                               // [2] producer -> consumers
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_yfree + 2);

  const int tid = threadIdx.x;
  const int blocks_per_b = D / C::kCh;
  const int b = blockIdx.x / blocks_per_b;
  const int d0 = (blockIdx.x % blocks_per_b) * C::kCh;
  const int ntiles = (T + C::kRows - 1) / C::kRows;
  constexpr int kAPitch = C::kBoxCols * C::kEsz;
  constexpr int kXPitch = C::kCh * C::kEsz;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], C::kConsumers);
    }
    mbar_init(&s_yfree[0], 1);
    mbar_init(&s_yfree[1], 1);
    *s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (tid >= C::kConsumers) {
    // ---------------------------------------------------------------- producer
    if (tid == C::kConsumers) {
      umma::tma_prefetch_desc(&map_a);
      umma::tma_prefetch_desc(&map_x);
      umma::tma_prefetch_desc(&map_y);
      auto issue_tile = [&](int tile) {
        const int s = tile % C::kStages;
        unsigned char* sa = s_stage + s * C::kStageBytes;
        mbar_arrive_expect_tx(&s_full[s], C::kStageBytes);
#pragma unroll
        for (int bx = 0; bx < C::kNumBox; ++bx)
          umma::tma_load_3d(sa + bx * (C::kRows * C::kBoxCols * C::kEsz), &map_a,
                            d0 * N + bx * C::kBoxCols, tile * C::kRows, b, &s_full[s]);
        umma::tma_load_3d(sa + C::kABytes, &map_x, d0, tile * C::kRows, b, &s_full[s]);
      };
      for (int i = 0; i < C::kStages && i < ntiles; ++i) issue_tile(i);
      for (int tile = 0; tile < ntiles; ++tile) {
        const int s = tile % C::kStages;
        // every consumer has finished reading stage s and staging y for `tile`
        if (!mbar_wait_abortable(&s_empty[s], (tile / C::kStages) & 1, s_abort)) break;
        umma::tma_store_3d(&map_y, d0, tile * C::kRows, b, s_y + (tile & 1) * C::kXBytes);
        bulk_commit();
        if (tile + C::kStages < ntiles) issue_tile(tile + C::kStages);
        // the store of the previous tile has left its staging buffer: hand it back
        bulk_wait_read<1>();
        if (tile >= 1) mbar_arrive(&s_yfree[(tile - 1) & 1]);
      }
      bulk_wait_all<0>();
      if (*s_abort && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT);
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int ch = tid / C::kLpc, sub = tid % C::kLpc;
  const int d = d0 + ch;
  const int e = ch * N + sub * NPT;   // this thread's elements inside a row of the `a` tile
  const int a_off = (e / C::kBoxCols) * (C::kRows * C::kBoxCols * C::kEsz) + (e % C::kBoxCols) * C::kEsz;
  constexpr int kPairs = NPT / 2;
  uint64_t h2[kPairs], b2[kPairs], c2[kPairs];
#pragma unroll
  for (int p = 0; p < kPairs; ++p) {
    const int n = sub * NPT + 2 * p;
    b2[p] = umma::f2_pack(E::ld(bvec, d * N + n), E::ld(bvec, d * N + n + 1));
    c2[p] = umma::f2_pack(E::ld(cvec, d * N + n), E::ld(cvec, d * N + n + 1));
    const size_t hi = (size_t(b) * D + d) * N + n;
    h2[p] = h0 ? umma::f2_pack(h0[hi], h0[hi + 1]) : umma::f2_pack(0.f, 0.f);
  }
  // After the transposing reduction a lane holds kKeep consecutive steps of a
  // group of four, starting at q_base; lanes with dup != 0 hold duplicates.
  constexpr int kXRounds = C::kLpc >= 4 ? 2 : (C::kLpc == 2 ? 1 : 0);
  constexpr int kKeep = 4 >> kXRounds;
  const int q_base = (kXRounds >= 1 && (sub & 1) ? 2 : 0) + (kXRounds >= 2 && (sub & 2) ? 1 : 0);
  const bool dup = (sub >> kXRounds) != 0;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int s = tile % C::kStages;
    const int rows = min(C::kRows, T - tile * C::kRows);
    bool ok = mbar_wait_abortable(&s_full[s], (tile / C::kStages) & 1, s_abort);
    if (ok && tile >= 2) ok = mbar_wait_abortable(&s_yfree[tile & 1], ((tile >> 1) - 1) & 1, s_abort);
    if (!ok) return;
    const unsigned char* sa = s_stage + s * C::kStageBytes + a_off;
    const unsigned char* sx = s_stage + s * C::kStageBytes + C::kABytes + ch * C::kEsz;
    unsigned char* sy = s_y + (tile & 1) * C::kXBytes;

    float av[2][4][NPT], xv[2][4];
    auto load_group = [&](int buf, int r0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        load_row<DTYPE, NPT>(sa + (r0 + q) * kAPitch, av[buf][q]);
        xv[buf][q] = E::ld(sx + (r0 + q) * kXPitch, 0);
      }
    };
    // Four steps from registers.  `limit` = number of valid steps in the group
    // (4 everywhere except in the ragged last tile, where the branch-free body
    // is replaced by a guarded one so that steps past T never touch the state).
    auto group = [&](int cur, int r0, auto full_tag, int limit) {
      constexpr bool kFull = decltype(full_tag)::value;
      float yv[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (kFull || q < limit) {
          const uint64_t x2 = umma::f2_pack(xv[cur][q], xv[cur][q]);
          uint64_t acc = umma::f2_pack(0.f, 0.f);
#pragma unroll
          for (int p = 0; p < kPairs; ++p) {
            const uint64_t a2 = umma::f2_pack(av[cur][q][2 * p], av[cur][q][2 * p + 1]);
            h2[p] = umma::f2_fma(a2, h2[p], umma::f2_mul(b2[p], x2));
            acc = umma::f2_fma(c2[p], h2[p], acc);
          }
          float lo, hi;
          umma::f2_unpack(acc, lo, hi);
          yv[q] = lo + hi;
        } else {
          yv[q] = 0.f;
        }
      }
      // transposing reduction over the lanes of a channel
      if constexpr (kXRounds >= 1) {
        const bool up = sub & 1;
        const float s0 = up ? yv[0] : yv[2], s1 = up ? yv[1] : yv[3];
        const float k0 = up ? yv[2] : yv[0], k1 = up ? yv[3] : yv[1];
        yv[0] = k0 + __shfl_xor_sync(0xffffffffu, s0, 1);
        yv[1] = k1 + __shfl_xor_sync(0xffffffffu, s1, 1);
      }
      if constexpr (kXRounds >= 2) {
        const bool up = sub & 2;
        const float s0 = up ? yv[0] : yv[1];
        const float k0 = up ? yv[1] : yv[0];
        yv[0] = k0 + __shfl_xor_sync(0xffffffffu, s0, 2);
      }
#pragma unroll
      for (int off = 1 << kXRounds; off < C::kLpc; off <<= 1) {   // lanes beyond four: plain butterfly
#pragma unroll
        for (int j = 0; j < kKeep; ++j) yv[j] += __shfl_xor_sync(0xffffffffu, yv[j], off);
      }
      if (!dup) {
#pragma unroll
        for (int j = 0; j < kKeep; ++j) E::st(sy + (r0 + q_base + j) * kXPitch, ch, yv[j]);
      }
    };
    load_group(0, 0);
    if (rows == C::kRows) {
#pragma unroll
      for (int gi = 0; gi < C::kRows / 4; ++gi) {
        if (gi + 1 < C::kRows / 4) load_group((gi & 1) ^ 1, gi * 4 + 4);   // next four steps' operands
        group(gi & 1, gi * 4, std::true_type{}, 4);
      }
    } else {
#pragma unroll 1
      for (int gi = 0; gi * 4 < rows; ++gi) {
        if (gi > 0) load_group(0, gi * 4);
        group(0, gi * 4, std::false_type{}, rows - gi * 4);
      }
    }
    fence_proxy_async_smem();      // staged y rows -> visible to the TMA store
    mbar_arrive(&s_empty[s]);      // stage s and this tile's y are the producer's now
  }
  if (hT) {
#pragma unroll
    for (int p = 0; p < kPairs; ++p) {
      float lo, hi;
      umma::f2_unpack(h2[p], lo, hi);
      const size_t hi_idx = (size_t(b) * D + d) * N + sub * NPT + 2 * p;
      hT[hi_idx] = lo;
      hT[hi_idx + 1] = hi;
    }
  }
}

template <int DTYPE, int N, int NPT>
int launch_scan_tma(const void* a, const void* x, const void* b, const void* c, const float* h0,
                    void* y, float* hT, int B, int T, int D, int* dev_status, cudaStream_t st) {
  using C = FastCfg<DTYPE, N, NPT>;
  CUtensorMap ma, mx, my;
  const bool bf = DTYPE == CB2_BF16;
  int rc = umma::make_map_3d(&ma, a, bf, uint64_t(D) * N, T, B, C::kBoxCols, C::kRows);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mx, x, bf, D, T, B, C::kCh, C::kRows);
  if (rc == CB2_OK) rc = umma::make_map_3d(&my, y, bf, D, T, B, C::kCh, C::kRows);
  if (rc != CB2_OK) return rc;
  auto kern = diag_scan_tma_kernel<DTYPE, N, NPT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  kern<<<B * (D / C::kCh), C::kThreads, C::kSmem, st>>>(ma, mx, my, b, c, h0, hT, T, D, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

// n per thread on the fast path: 4 (8 n per thread was measured and is no faster).
inline int scan_npt() { return 4; }

// ---------------------------------------------------------------------------
// `a` shared over n ([B,T,D]), fast path (D a multiple of 32).  With one decay
// per channel the N states are all multiples of ONE scalar recurrence:
//   h_t[n] = b[n] * G_t + P_t * h0[n],   G_t = a_t G_{t-1} + x_t,   P_t = a_t P_{t-1}
// so  y_t = (sum_n c[n] b[n]) * G_t + (sum_n c[n] h0[n]) * P_t  needs a few FMAs
// per step instead of 2N.  Traffic is a, x, y only (6 bytes of bf16 per (b,t,d)).
//
// Only B*D/32 warps' worth of channels exist, too few to hide latency, so the
// T axis is cut into 64-step tiles dealt round-robin to the four consumer warps
// of a CTA (lane = channel).  A warp first runs its tile from the identity
// (local G_t, P_t kept in registers), then receives the carry (G, P) at the
// tile's start from the owner of the previous tile through shared memory and an
// mbarrier, publishes its own carry-out with two FMAs — the only serial step —
// and finally corrects and stores its 64 outputs.  A producer warp streams the
// a / x tiles through an 8-stage ring with tiled TMA and stores the y tiles.
// ---------------------------------------------------------------------------
template <int DTYPE>
struct SharedACfg {
  static constexpr int kEsz = Elem<DTYPE>::kSize;
  static constexpr int kCh = 32;
  static constexpr int kRows = 64;
  static constexpr int kWarps = 4;                          // consumer warps = tiles in flight
  static constexpr int kYBufs = 8;                          // y staging tiles (two per consumer warp)
  static constexpr int kStages = 8;
  static constexpr int kThreads = (kWarps + 1) * 32;
  static constexpr int kTileBytes = kRows * kCh * kEsz;     // one operand, one tile
  static constexpr int kStageBytes = 2 * kTileBytes;        // a | x
  static constexpr int kNumBars = 2 * kStages + kYBufs + kWarps;
  static constexpr int kSmem = kStages * kStageBytes + kYBufs * kTileBytes + kWarps * 2 * kCh * 4 +
                               kNumBars * 8 + 16 + 128;
};

template <int DTYPE>
__global__ void __launch_bounds__(SharedACfg<DTYPE>::kThreads)
diag_scan_shared_a_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_x,
                          const __grid_constant__ CUtensorMap map_y, const void* __restrict__ bvec,
                          const void* __restrict__ cvec, const float* __restrict__ h0,
                          float* __restrict__ hT, int T, int D, int N, int* dev_status) {
  using C = SharedACfg<DTYPE>;
  using E = Elem<DTYPE>;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* s_stage = smem;
  unsigned char* s_y = smem + C::kStages * C::kStageBytes;                    // kYBufs staging tiles
  float* s_carry = reinterpret_cast<float*>(s_y + C::kYBufs * C::kTileBytes); // [kWarps][2][32]
  uint64_t* s_full = reinterpret_cast<uint64_t*>(s_carry + C::kWarps * 2 * C::kCh);
  uint64_t* s_empty = s_full + C::kStages;
  uint64_t* s_yfree = s_empty + C::kStages;     // [kYBufs] producer -> consumers: staging tile reusable
  uint64_t* s_cbar = s_yfree + C::kYBufs;       // [kWarps] carry of warp w published
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_cbar + C::kWarps);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blocks_per_b = D / C::kCh;
  const int b = blockIdx.x / blocks_per_b;
  const int d0 = (blockIdx.x % blocks_per_b) * C::kCh;
  const int ntiles = (T + C::kRows - 1) / C::kRows;
  constexpr int kPitch = C::kCh * C::kEsz;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 32);
    }
    for (int w = 0; w < C::kYBufs; ++w) mbar_init(&s_yfree[w], 1);
    for (int w = 0; w < C::kWarps; ++w) mbar_init(&s_cbar[w], 32);
    *s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == C::kWarps) {
    if (lane == 0) {  // producer
      umma::tma_prefetch_desc(&map_a);
      umma::tma_prefetch_desc(&map_x);
      umma::tma_prefetch_desc(&map_y);
      auto issue_tile = [&](int tile) {
        const int s = tile % C::kStages;
        unsigned char* st = s_stage + s * C::kStageBytes;
        mbar_arrive_expect_tx(&s_full[s], C::kStageBytes);
        umma::tma_load_3d(st, &map_a, d0, tile * C::kRows, b, &s_full[s]);
        umma::tma_load_3d(st + C::kTileBytes, &map_x, d0, tile * C::kRows, b, &s_full[s]);
      };
      for (int i = 0; i < C::kStages && i < ntiles; ++i) issue_tile(i);
      for (int tile = 0; tile < ntiles; ++tile) {
        const int s = tile % C::kStages;
        if (!mbar_wait_abortable(&s_empty[s], (tile / C::kStages) & 1, s_abort)) break;
        umma::tma_store_3d(&map_y, d0, tile * C::kRows, b, s_y + (tile % C::kYBufs) * C::kTileBytes);
        bulk_commit();
        if (tile + C::kStages < ntiles) issue_tile(tile + C::kStages);
        // all but the newest 3 stores have left their staging tiles; a tile is reused
        // kYBufs tiles later, so consumers never wait on a neighbour's store
        bulk_wait_read<3>();
        if (tile >= 3) mbar_arrive(&s_yfree[(tile - 3) % C::kYBufs]);
      }
      bulk_wait_all<0>();
      if (*s_abort && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT);
    }
    return;
  }

  // consumer warps: lane = channel, warp w owns tiles w, w + kWarps, ...
  const int d = d0 + lane;
  float cb = 0.f, ch0 = 0.f;
  for (int n = 0; n < N; ++n) {
    const float cn = E::ld(cvec, d * N + n);
    cb = fmaf(cn, E::ld(bvec, d * N + n), cb);
    if (h0) ch0 = fmaf(cn, h0[(size_t(b) * D + d) * N + n], ch0);
  }
  const int prev = (warp + C::kWarps - 1) % C::kWarps;
  float g_end = 0.f, p_end = 1.f;   // carry after this warp's latest tile
  for (int tile = warp, round = 0; tile < ntiles; tile += C::kWarps, ++round) {
    const int s = tile % C::kStages;
    const int rows = min(C::kRows, T - tile * C::kRows);
    bool ok = mbar_wait_abortable(&s_full[s], (tile / C::kStages) & 1, s_abort);
    if (!__all_sync(0xffffffffu, ok)) return;
    const unsigned char* sa = s_stage + s * C::kStageBytes + lane * C::kEsz;
    const unsigned char* sx = sa + C::kTileBytes;
    // pass 1: the tile from the identity; rows past T act as the identity map (a=1, x=0)
    float gl[C::kRows], pl[C::kRows];
    float g = 0.f, p = 1.f;
#pragma unroll
    for (int r0 = 0; r0 < C::kRows; r0 += 8) {
      float av[8], xv[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const bool in = r0 + q < rows;
        av[q] = in ? E::ld(sa + (r0 + q) * kPitch, 0) : 1.f;
        xv[q] = in ? E::ld(sx + (r0 + q) * kPitch, 0) : 0.f;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        g = fmaf(av[q], g, xv[q]);
        p *= av[q];
        gl[r0 + q] = g;
        pl[r0 + q] = p;
      }
    }
    // carry-in from the owner of the previous tile
    float g_in = 0.f, p_in = 1.f;
    if (tile > 0) {
      const int pr = warp == 0 ? round - 1 : round;   // round in which `prev` published it
      ok = mbar_wait_abortable(&s_cbar[prev], pr & 1, s_abort);
      if (!__all_sync(0xffffffffu, ok)) return;
      g_in = s_carry[(prev * 2 + 0) * C::kCh + lane];
      p_in = s_carry[(prev * 2 + 1) * C::kCh + lane];
    }
    g_end = fmaf(pl[C::kRows - 1], g_in, gl[C::kRows - 1]);
    p_end = pl[C::kRows - 1] * p_in;
    s_carry[(warp * 2 + 0) * C::kCh + lane] = g_end;
    s_carry[(warp * 2 + 1) * C::kCh + lane] = p_end;
    mbar_arrive(&s_cbar[warp]);  // release: the next tile's owner may go on
    // pass 2: corrected outputs into this warp's staging tile
    if (tile >= C::kYBufs) {
      ok = mbar_wait_abortable(&s_yfree[tile % C::kYBufs], ((tile / C::kYBufs) - 1) & 1, s_abort);
      if (!__all_sync(0xffffffffu, ok)) return;
    }
    unsigned char* sy = s_y + (tile % C::kYBufs) * C::kTileBytes;
    const float cg = cb * g_in, cp = ch0 * p_in;
#pragma unroll
    for (int r = 0; r < C::kRows; ++r) {
      // y = cb*(gl + pl*g_in) + ch0*(pl*p_in)
      const float yv = fmaf(cb, gl[r], pl[r] * (cg + cp));
      E::st(sy + r * kPitch, lane, yv);
    }
    fence_proxy_async_smem();
    mbar_arrive(&s_empty[s]);
  }
  // the owner of the last tile holds the final carry
  if (hT && warp == (ntiles - 1) % C::kWarps) {
    for (int n = 0; n < N; ++n) {
      const size_t i = (size_t(b) * D + d) * N + n;
      hT[i] = fmaf(E::ld(bvec, d * N + n), g_end, h0 ? p_end * h0[i] : 0.f);
    }
  }
}

template <int DTYPE>
int launch_scan_shared_a(const void* a, const void* x, const void* b, const void* c, const float* h0,
                         void* y, float* hT, int B, int T, int D, int N, int* dev_status, cudaStream_t st) {
  using C = SharedACfg<DTYPE>;
  CUtensorMap ma, mx, my;
  const bool bf = DTYPE == CB2_BF16;
  int rc = umma::make_map_3d(&ma, a, bf, D, T, B, C::kCh, C::kRows);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mx, x, bf, D, T, B, C::kCh, C::kRows);
  if (rc == CB2_OK) rc = umma::make_map_3d(&my, y, bf, D, T, B, C::kCh, C::kRows);
  if (rc != CB2_OK) return rc;
  auto kern = diag_scan_shared_a_kernel<DTYPE>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  kern<<<B * (D / C::kCh), C::kThreads, C::kSmem, st>>>(ma, mx, my, b, c, h0, hT, T, D, N, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

// `a` shared over n, generic path: one thread per (b, channel) keeps all N states.
template <int DTYPE, int N>
__global__ void __launch_bounds__(128)
diag_scan_bcast_kernel(const void* __restrict__ a, const void* __restrict__ x,
                       const void* __restrict__ bvec, const void* __restrict__ cvec,
                       const float* __restrict__ h0, void* __restrict__ y,
                       float* __restrict__ hT, int B, int T, int D) {
  using E = Elem<DTYPE>;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * D) return;
  const int b = idx / D, d = idx % D;
  float h[N], bw[N], cw[N];
#pragma unroll
  for (int n = 0; n < N; ++n) {
    bw[n] = E::ld(bvec, d * N + n);
    cw[n] = E::ld(cvec, d * N + n);
    h[n] = h0 ? h0[(size_t(b) * D + d) * N + n] : 0.f;
  }
  const size_t base = size_t(b) * T * D + d;
#pragma unroll 8
  for (int t = 0; t < T; ++t) {
    const float av = E::ld(a, 0 + (base + size_t(t) * D));
    const float xv = E::ld(x, 0 + (base + size_t(t) * D));
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      h[n] = fmaf(av, h[n], bw[n] * xv);
      acc = fmaf(cw[n], h[n], acc);
    }
    E::st(y, base + size_t(t) * D, acc);
  }
  if (hT) {
#pragma unroll
    for (int n = 0; n < N; ++n) hT[(size_t(b) * D + d) * N + n] = h[n];
  }
}

template <int DTYPE, int N>
int launch_scan(const void* a, const void* x, const void* b, const void* c, const float* h0,
                void* y, float* hT, int B, int T, int D, int a_bcast_n, int* dev_status,
                cudaStream_t st) {
  using C = ScanCfg<DTYPE, N>;
  if (N == 1) a_bcast_n = 1;   // [B,T,D,1] is [B,T,D]: the collapsed-recurrence kernel applies
  if (a_bcast_n) {
    if (D % 32 == 0 && aligned16(a) && aligned16(x) && aligned16(y))
      return launch_scan_shared_a<DTYPE>(a, x, b, c, h0, y, hT, B, T, D, N, dev_status, st);
    const int total = B * D;
    diag_scan_bcast_kernel<DTYPE, N><<<(total + 127) / 128, 128, 0, st>>>(a, x, b, c, h0, y, hT,
                                                                         B, T, D);
    CB2_LAUNCH_CHECK();
    return CB2_OK;
  }
  if ((size_t(D) * N * C::kEsz) % 16 || (size_t(D) * C::kEsz) % 16) return CB2_BAD_SHAPE;
  if constexpr (N >= 4) {
    if (D % 32 == 0) {
      if constexpr (N >= 8) {
        if (scan_npt() == 8)
          return launch_scan_tma<DTYPE, N, 8>(a, x, b, c, h0, y, hT, B, T, D, dev_status, st);
      }
      return launch_scan_tma<DTYPE, N, 4>(a, x, b, c, h0, y, hT, B, T, D, dev_status, st);
    }
  }
  auto kern = diag_scan_kernel<DTYPE, N>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) !=
      cudaSuccess)
    return CB2_LAUNCH_FAIL;
  const int blocks_per_b = (D + C::kCh - 1) / C::kCh;
  kern<<<B * blocks_per_b, C::kThreads, C::kSmem, st>>>(
      static_cast<const unsigned char*>(a), static_cast<const unsigned char*>(x), b, c, h0,
      static_cast<unsigned char*>(y), hT, T, D, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

template <int DTYPE>
int dispatch_n(const void* a, const void* x, const void* b, const void* c, const float* h0,
               void* y, float* hT, int B, int T, int D, int N, int a_bcast_n, int* dev_status,
               cudaStream_t st) {
#define CB2_SCAN_CASE(NN) \
  case NN:                \
    return launch_scan<DTYPE, NN>(a, x, b, c, h0, y, hT, B, T, D, a_bcast_n, dev_status, st);
  switch (N) {
    CB2_SCAN_CASE(1)
    CB2_SCAN_CASE(2)
    CB2_SCAN_CASE(4)
    CB2_SCAN_CASE(8)
    CB2_SCAN_CASE(16)
    CB2_SCAN_CASE(32)
    default:
      return CB2_BAD_SHAPE;
  }
#undef CB2_SCAN_CASE
}

}  // namespace
}  // namespace cb2

extern "C" int cb2_diag_scan_fwd(const void* a, const void* x, const void* b, const void* c,
                                 const float* h0, void* y, float* hT, int B, int T, int D, int N,
                                 int a_bcast_n, int dtype, int* dev_status, void* stream) {
  if (!a || !x || !b || !c || !y) return CB2_NULL_PTR;
  if (B <= 0 || T <= 0 || D <= 0 || N <= 0) return CB2_BAD_SHAPE;
  if (!cb2::aligned16(a) || !cb2::aligned16(x) || !cb2::aligned16(y)) return CB2_BAD_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CB2_BF16)
    return cb2::dispatch_n<CB2_BF16>(a, x, b, c, h0, y, hT, B, T, D, N, a_bcast_n, dev_status, st);
  if (dtype == CB2_F32)
    return cb2::dispatch_n<CB2_F32>(a, x, b, c, h0, y, hT, B, T, D, N, a_bcast_n, dev_status, st);
  return CB2_UNSUPPORTED_DTYPE;
}
