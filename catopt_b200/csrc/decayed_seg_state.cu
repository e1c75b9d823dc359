// End states of sequence segments for the chunk-parallel form of decayed attention
// (bf16, tensor cores).  With fewer heads than SMs one CTA per head leaves most of the
// GPU idle, because the state carry of the recurrence the reference spells in
// lab/probes/retnet_baseline_probe.py:77-110 serialises the sequence.  The carry is
// an affine scan of the state (`decay_state_lift`, catopt_carriers/om.py:3850-3866),
// so a head can be cut into segments that run at the same time once every segment
// knows the state it starts from:
//
//   1. this file, kernel 1: the state each segment (but the last) would END in when
//      started from zero,   E_s = sum_r g^(L-1-r) K[r]^T V[r]   over the segment's L rows
//      (one accumulation in tensor memory; only decaying powers appear, and bf16
//      keeps their relative precision down to underflow, where the term is nil);
//   2. this file, kernel 2: the start states by the scan  S_s = g^L S_(s-1) + E_(s-1),
//      S_0 = 0, in fp32, written where the attention kernel expects a segment's
//      incoming state (skipped when there are at most four pieces to fold: the attention
//      CTAs then fold the end states themselves, and the pre-pass cuts every segment into
//      shorter pieces so that it fills the GPU too);
//   3. decayed_chunk_tc.cu with all segments launched at once, each starting from its
//      S_s instead of waiting for its predecessor.
// K and V are read once more than in the one-pass form (6 units of traffic instead of
// 4), which costs nothing while the GPU is mostly idle.
//
// Kernel 1: CTA = (head, segment); K_i / V_i tiles of 128 rows stream through a 3-slot
// ring by TMA; 8 warps scale the rows of K_i by g^(L-1-r) in place; one thread issues
// E += Kw_i^T V_i (both operands MN-major from their tiles); the accumulator is read
// out once at the end.  Every wait is bounded.
#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kSC = 128;
constexpr int kSsSlots = 3;
constexpr int kSsThreads = 320;
constexpr int kSsCompute = 256;
constexpr uint32_t kSsTile = umma::kTileBytes;            // 32 KiB
constexpr uint32_t kSsStage = 2 * kSsTile;                // K_i | V_i
constexpr uint32_t kSsOffBars = kSsSlots * kSsStage;
constexpr int kSsNumBars = 3 * kSsSlots + 1;
constexpr uint32_t kSsOffMisc = kSsOffBars + kSsNumBars * 8;
constexpr uint32_t kSsSmem = kSsOffMisc + 16 + 1024;

__global__ void __launch_bounds__(kSsThreads, 1)
decayed_seg_state_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const float* __restrict__ gamma, int H, int n_bh, int chunks_per_seg,
                         float* __restrict__ seg_state, int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSsOffBars);
  uint64_t* full = bars;                     // TMA -> scaling group
  uint64_t* kw_ready = bars + kSsSlots;      // scaling group -> MMA (256 arrivals)
  uint64_t* empty = bars + 2 * kSsSlots;     // MMA -> TMA
  uint64_t* acc_ready = bars + 3 * kSsSlots;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kSsOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kSsOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x % n_bh, seg = blockIdx.x / n_bh;
  const int chunk0 = seg * chunks_per_seg;
  const float g = gamma[bh % H];
  const int L = chunks_per_seg * kSC;

  if (tid == 0) {
    for (int s = 0; s < kSsSlots; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&kw_ready[s], kSsCompute);
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
      umma::tma_prefetch_desc(&map_k);
      umma::tma_prefetch_desc(&map_v);
      for (int i = 0; i < chunks_per_seg; ++i) {
        const int slot = i % kSsSlots, use = i / kSsSlots;
        if (use > 0 && !mbar_wait_abortable(&empty[slot], (use - 1) & 1, s_abort)) break;
        unsigned char* dst = smem + slot * kSsStage;
        const int row = (chunk0 + i) * kSC;
        mbar_arrive_expect_tx(&full[slot], 2 * kSsTile);
        umma::tma_load_3d(dst, &map_k, 0, row, bh, &full[slot]);
        umma::tma_load_3d(dst + umma::kSubTileBytes, &map_k, 64, row, bh, &full[slot]);
        umma::tma_load_3d(dst + kSsTile, &map_v, 0, row, bh, &full[slot]);
        umma::tma_load_3d(dst + kSsTile + umma::kSubTileBytes, &map_v, 64, row, bh, &full[slot]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_nn = umma::instr_desc_bf16(128, 128, true, true);
      const uint32_t ring = smem_u32(smem);
      bool ok = true;
      for (int i = 0; i < chunks_per_seg; ++i) {
        const int slot = i % kSsSlots, use = i / kSsSlots;
        ok = mbar_wait_abortable(&kw_ready[slot], use & 1, s_abort);
        if (!ok) break;
        umma::fence_after_sync();
        const uint32_t k_addr = ring + slot * kSsStage, v_addr = k_addr + kSsTile;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16(tmem, umma::desc_mnmajor(k_addr, ks), umma::desc_mnmajor(v_addr, ks), idesc_nn,
                         i > 0 || ks > 0);
        umma::mma_commit(&empty[slot]);
      }
      if (ok) umma::mma_commit(acc_ready);
    }
  } else {
    // thread = (row r of the chunk, column half of K)
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q4 * 32 + lane;
    for (int i = 0; i < chunks_per_seg; ++i) {
      const int slot = i % kSsSlots, use = i / kSsSlots;
      bool ok = mbar_wait_abortable(&full[slot], use & 1, s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      // weight of row r of chunk i: g^(L-1-R), R its index within the segment
      const float w = powf(g, float(L - 1 - (i * kSC + r)));
      unsigned char* k_tile = smem + slot * kSsStage;
      uint4 x[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        x[j] = *reinterpret_cast<const uint4*>(k_tile + umma::tile_chunk_offset(r, half * 64 + j * 8));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        x[j].x = pack_bf16x2(bf16lo_to_f32(x[j].x) * w, bf16hi_to_f32(x[j].x) * w);
        x[j].y = pack_bf16x2(bf16lo_to_f32(x[j].y) * w, bf16hi_to_f32(x[j].y) * w);
        x[j].z = pack_bf16x2(bf16lo_to_f32(x[j].z) * w, bf16hi_to_f32(x[j].z) * w);
        x[j].w = pack_bf16x2(bf16lo_to_f32(x[j].w) * w, bf16hi_to_f32(x[j].w) * w);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(k_tile + umma::tile_chunk_offset(r, half * 64 + j * 8)) = x[j];
      fence_proxy_async_smem();
      mbar_arrive(&kw_ready[slot]);
    }
    // E[e][f]: TMEM lane = e, column = f  ->  float[128][128] of this (segment, head)
    bool ok = mbar_wait_abortable(acc_ready, 0, s_abort);
    if (__all_sync(0xffffffffu, ok)) {
      umma::fence_after_sync();
      const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
      float4* dst = reinterpret_cast<float4*>(seg_state + (size_t(seg) * n_bh + bh) * (kSC * kSC) + r * kSC + half * 64);
      uint32_t va[32], vb[32];
      umma::tmem_ld32(lane_base + half * 64, va);
      umma::tmem_ld32(lane_base + half * 64 + 32, vb);
      umma::tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dst[j] = make_float4(__uint_as_float(va[4 * j]), __uint_as_float(va[4 * j + 1]),
                             __uint_as_float(va[4 * j + 2]), __uint_as_float(va[4 * j + 3]));
        dst[8 + j] = make_float4(__uint_as_float(vb[4 * j]), __uint_as_float(vb[4 * j + 1]),
                                 __uint_as_float(vb[4 * j + 2]), __uint_as_float(vb[4 * j + 3]));
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

// S_s = g^L S_(s-1) + E_(s-1), in place: slot s-1 holds E_(s-1) on entry and S_s on exit.
__global__ void __launch_bounds__(256)
decayed_seg_scan_kernel(float* __restrict__ seg_state, const float* __restrict__ gamma, int H, int n_bh,
                        int n_seg, int L) {
  const int bh = blockIdx.y;
  const int idx = blockIdx.x * 256 + threadIdx.x;      // element of the 128 x 128 state
  const float gL = powf(gamma[bh % H], float(L));
  float acc = 0.f;
  for (int s = 1; s < n_seg; ++s) {
    float* p = seg_state + (size_t(s - 1) * n_bh + bh) * (kSC * kSC) + idx;
    acc = fmaf(gL, acc, *p);
    *p = acc;
  }
}

}  // namespace

// Phase 1 and 2 of the chunk-parallel form.  sub == 0: afterwards slot s-1 of seg_state holds the
// state segment s starts from (s = 1 .. n_seg-1).  sub > 0: every segment but the last is cut
// into `sub` pieces, slot p holds the end state (from zero) of piece p, and the attention kernel
// folds the pieces before a segment itself (no scan launch).
int decayed_seg_states_run(const void* k, const void* v, const float* gamma, int B, int H, int T, int dk,
                           int dv, int n_seg, int sub, float* seg_state, int* dev_status, cudaStream_t st) {
  const uint64_t heads = uint64_t(B) * H;
  const int n_bh = B * H;
  const int nchunk = (T + kSC - 1) / kSC;
  const int per = nchunk / n_seg;
  const int pieces = (n_seg - 1) * (sub > 0 ? sub : 1);
  const int piece_chunks = sub > 0 ? per / sub : per;
  CUtensorMap mk, mv;
  int rc = umma::make_map_3d(&mk, k, true, dk, T, heads, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mv, v, true, dv, T, heads, 64, 128, true);
  if (rc != CB2_OK) return rc;
  if (cudaFuncSetAttribute(decayed_seg_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           int(kSsSmem)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  decayed_seg_state_kernel<<<unsigned(n_bh * pieces), kSsThreads, kSsSmem, st>>>(mk, mv, gamma, H, n_bh, piece_chunks,
                                                                                seg_state, dev_status);
  CB2_LAUNCH_CHECK();
  if (sub > 0) return CB2_OK;
  decayed_seg_scan_kernel<<<dim3(kSC * kSC / 256, unsigned(n_bh)), 256, 0, st>>>(seg_state, gamma, H, n_bh, n_seg,
                                                                                 per * kSC);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
