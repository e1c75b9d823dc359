// Chunked decayed attention on the 5th-generation tensor cores (bf16 tensors,
// chunk = dk = dv = 128): one CTA per (batch, head) walks the chunks in order
// and keeps the fp32 inter-chunk state in tensor memory for the whole sequence.
//
// Per chunk i (C = 128 rows, g = gamma of the head):
//   MMA1  S  = Q_i K_i^T                                  (TMEM cols   0..127)
//   WG    P  = bf16( S . tril(g^(r-c)) )  -> smem ;  K_i <- K_i . g^(C-1-r) in place
//   MMA2  O1 = P V_i                                       (TMEM cols 128..255)
//   MMA3  O2 = Q_i Sb_i        (Sb_i = bf16 copy of the state, i > 0)   (256..383)
//   WG    o_i = (O1 + g^(r+1) O2) / scale  -> global
//   MMA4  St = [g^C St] + Kw_i^T V_i                       (TMEM cols 384..511)
//   WG    Sb_{i+1} = bf16(St) -> smem ;  St <- g^C St  (ready for the next MMA4)
// which is the state-carry recurrence the reference spells in
// lab/probes/retnet_baseline_probe.py:77-110 and equals its pairwise executor
// (decayed_lower.py:671-700) up to reassociation.  Only chunk-local powers of g
// appear.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer (and TMEM owner),
// warps 2..5 = the 128-thread compute group (thread = one TMEM lane = one row).
// Operand tiles (32 KiB each, K_i / Q_i / V_i in that order) stream through a
// 5-slot shared-memory ring with full/empty mbarriers; a slot is released by
// the tcgen05.commit of the last MMA that reads it, so up to two tiles of the
// next chunk are in flight while a chunk computes.  HBM traffic is exactly the
// algorithmic bytes: q, k, v read once, o written once.
#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kC = 128;                 // chunk rows = dk = dv
constexpr int kSlots = 5;
constexpr int kThreads = 192;
constexpr uint32_t kTile = umma::kTileBytes;      // 32 KiB
// shared memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffRing = 0;
constexpr uint32_t kOffP = kSlots * kTile;
constexpr uint32_t kOffSb = kOffP + kTile;
constexpr uint32_t kOffPow = kOffSb + kTile;                 // float[kC + 1]
constexpr uint32_t kOffBars = kOffPow + 528;                 // 8-byte aligned
constexpr int kNumBars = 2 * kSlots + 7;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;       // tmem base, abort flag
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;        // + alignment slack

// TMEM columns
constexpr uint32_t kColS = 0, kColO1 = 128, kColO2 = 256, kColSt = 384;

struct Bars {
  uint64_t* full;      // [kSlots] TMA -> MMA
  uint64_t* empty;     // [kSlots] MMA -> TMA
  uint64_t* s_ready;   // MMA1 done            (MMA -> WG)
  uint64_t* p_ready;   // P written            (WG -> MMA, 128 arrivals)
  uint64_t* kw_ready;  // K scaled in place    (WG -> MMA, 128)
  uint64_t* o_ready;   // MMA2+MMA3 done       (MMA -> WG)
  uint64_t* o_free;    // O1/O2 read out       (WG -> MMA, 128)
  uint64_t* st_ready;  // MMA4 done            (MMA -> WG)
  uint64_t* sb_ready;  // Sb written, St scaled (WG -> MMA, 128)
};

__global__ void __launch_bounds__(kThreads, 1)
decayed_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ o,
                  const float* __restrict__ gamma, int H, int T, float inv_scale, int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* s_pow = reinterpret_cast<float*>(smem + kOffPow);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 4);
  Bars B{bars, bars + kSlots, bars + 2 * kSlots, bars + 2 * kSlots + 1, bars + 2 * kSlots + 2,
         bars + 2 * kSlots + 3, bars + 2 * kSlots + 4, bars + 2 * kSlots + 5, bars + 2 * kSlots + 6};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x;
  const int nchunk = T / kC;
  const float g = gamma[bh % H];
  const uint32_t ring_addr = smem_u32(smem + kOffRing);
  const uint32_t p_addr = smem_u32(smem + kOffP);
  const uint32_t sb_addr = smem_u32(smem + kOffSb);

  if (tid == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&B.full[s], 1);
      mbar_init(&B.empty[s], 1);
    }
    mbar_init(B.s_ready, 1);
    mbar_init(B.p_ready, 128);
    mbar_init(B.kw_ready, 128);
    mbar_init(B.o_ready, 1);
    mbar_init(B.o_free, 128);
    mbar_init(B.st_ready, 1);
    mbar_init(B.sb_ready, 128);
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    umma::tmem_alloc(s_tmem, 512);
  }
  if (tid >= 64) {  // powers of gamma for this head: g^0 .. g^128
    const int j = tid - 64;
    s_pow[j] = powf(g, float(j));
    if (j == 0) s_pow[kC] = powf(g, float(kC));
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      umma::tma_prefetch_desc(&map_q);
      umma::tma_prefetch_desc(&map_k);
      umma::tma_prefetch_desc(&map_v);
      const int ntiles = 3 * nchunk;
      for (int t = 0; t < ntiles; ++t) {
        const int slot = t % kSlots, use = t / kSlots;
        if (use > 0 && !mbar_wait_abortable(&B.empty[slot], (use - 1) & 1, s_abort)) break;
        const int i = t / 3, which = t % 3;  // 0: K, 1: Q, 2: V
        const CUtensorMap* m = which == 0 ? &map_k : (which == 1 ? &map_q : &map_v);
        unsigned char* dst = smem + kOffRing + slot * kTile;
        const int row = bh * T + i * kC;
        mbar_arrive_expect_tx(&B.full[slot], kTile);
        umma::tma_load_2d(dst, m, 0, row, &B.full[slot]);
        umma::tma_load_2d(dst + umma::kSubTileBytes, m, 64, row, &B.full[slot]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_kk = umma::instr_desc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_kn = umma::instr_desc_bf16(128, 128, false, true);
      constexpr uint32_t idesc_nn = umma::instr_desc_bf16(128, 128, true, true);
      for (int i = 0; i < nchunk; ++i) {
        const uint32_t ph = i & 1;
        const int tk = 3 * i, tq = tk + 1, tv = tk + 2;
        const uint32_t k_addr = ring_addr + (tk % kSlots) * kTile;
        const uint32_t q_addr = ring_addr + (tq % kSlots) * kTile;
        const uint32_t v_addr = ring_addr + (tv % kSlots) * kTile;
        // MMA1: S = Q K^T
        if (!mbar_wait_abortable(&B.full[tk % kSlots], (tk / kSlots) & 1, s_abort)) break;
        if (!mbar_wait_abortable(&B.full[tq % kSlots], (tq / kSlots) & 1, s_abort)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16(tmem + kColS, umma::desc_kmajor(q_addr, ks), umma::desc_kmajor(k_addr, ks),
                         idesc_kk, ks > 0);
        umma::mma_commit(B.s_ready);
        // MMA2: O1 = P V
        if (!mbar_wait_abortable(B.p_ready, ph, s_abort)) break;
        if (!mbar_wait_abortable(&B.full[tv % kSlots], (tv / kSlots) & 1, s_abort)) break;
        if (i > 0 && !mbar_wait_abortable(B.o_free, (i - 1) & 1, s_abort)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16(tmem + kColO1, umma::desc_kmajor(p_addr, ks), umma::desc_mnmajor(v_addr, ks),
                         idesc_kn, ks > 0);
        // MMA3: O2 = Q Sb   (the state is zero before the first chunk)
        if (i > 0) {
          if (!mbar_wait_abortable(B.sb_ready, (i - 1) & 1, s_abort)) break;
          umma::fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma::mma_bf16(tmem + kColO2, umma::desc_kmajor(q_addr, ks),
                           umma::desc_mnmajor(sb_addr, ks), idesc_kn, ks > 0);
        }
        umma::mma_commit(B.o_ready);
        umma::mma_commit(&B.empty[tq % kSlots]);
        // MMA4: St (+)= Kw^T V
        if (!mbar_wait_abortable(B.kw_ready, ph, s_abort)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16(tmem + kColSt, umma::desc_mnmajor(k_addr, ks), umma::desc_mnmajor(v_addr, ks),
                         idesc_nn, (i > 0) || (ks > 0));
        umma::mma_commit(B.st_ready);
        umma::mma_commit(&B.empty[tk % kSlots]);
        umma::mma_commit(&B.empty[tv % kSlots]);
      }
    }
  } else {
    // ------------------------------------------------------------ compute group
    const int q4 = warp & 3;                 // TMEM lane quarter this warp may touch
    const int r = q4 * 32 + lane;            // row of the chunk / lane of TMEM
    const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
    const float g_row = s_pow[r + 1];        // g^(r+1)
    const float g_col = s_pow[kC - 1 - r];   // g^(C-1-r)
    const float g_chunk = s_pow[kC];         // g^C
    unsigned char* p_tile = smem + kOffP;
    unsigned char* sb_tile = smem + kOffSb;
    uint32_t v[32];
    for (int i = 0; i < nchunk; ++i) {
      const uint32_t ph = i & 1;
      bool ok = mbar_wait_abortable(B.s_ready, ph, s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      umma::fence_after_sync();
      // (a) P = bf16(S . decay), written K-major into the P tile
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        if (cb <= q4) {
          umma::tmem_ld32(lane_base + kColS + cb * 32, v);
          umma::tmem_wait_ld();
        }
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = cb * 32 + c8 * 8 + 2 * j;
            float lo = 0.f, hi = 0.f;
            if (cb <= q4) {
              if (c <= r) lo = __uint_as_float(v[c8 * 8 + 2 * j]) * s_pow[r - c];
              if (c + 1 <= r) hi = __uint_as_float(v[c8 * 8 + 2 * j + 1]) * s_pow[r - c - 1];
            }
            w[j] = pack_bf16x2(lo, hi);
          }
          *reinterpret_cast<uint4*>(p_tile + umma::tile_chunk_offset(r, cb * 32 + c8 * 8)) =
              make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      umma::fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(B.p_ready);
      // (b) K_i <- K_i . g^(C-1-r), in place (MMA1 has finished reading it)
      {
        unsigned char* k_tile = smem + kOffRing + ((3 * i) % kSlots) * kTile;
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const int col = ((jj & 7) ^ (r & 7)) * 8 + (jj >> 3) * 64;   // conflict-free chunk order
          uint4* pch = reinterpret_cast<uint4*>(k_tile + umma::tile_chunk_offset(r, col));
          uint4 x = *pch;
          x.x = pack_bf16x2(bf16lo_to_f32(x.x) * g_col, bf16hi_to_f32(x.x) * g_col);
          x.y = pack_bf16x2(bf16lo_to_f32(x.y) * g_col, bf16hi_to_f32(x.y) * g_col);
          x.z = pack_bf16x2(bf16lo_to_f32(x.z) * g_col, bf16hi_to_f32(x.z) * g_col);
          x.w = pack_bf16x2(bf16lo_to_f32(x.w) * g_col, bf16hi_to_f32(x.w) * g_col);
          *pch = x;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(B.kw_ready);
      // (c) o_i = (O1 + g^(r+1) O2) / scale
      ok = mbar_wait_abortable(B.o_ready, ph, s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      umma::fence_after_sync();
      {
        __nv_bfloat16* orow = o + (size_t(bh) * T + size_t(i) * kC + r) * kC;
        uint32_t v2[32];
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          umma::tmem_ld32(lane_base + kColO1 + cb * 32, v);
          if (i > 0) umma::tmem_ld32(lane_base + kColO2 + cb * 32, v2);
          umma::tmem_wait_ld();
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float lo = __uint_as_float(v[c8 * 8 + 2 * j]), hi = __uint_as_float(v[c8 * 8 + 2 * j + 1]);
              if (i > 0) {
                lo = fmaf(g_row, __uint_as_float(v2[c8 * 8 + 2 * j]), lo);
                hi = fmaf(g_row, __uint_as_float(v2[c8 * 8 + 2 * j + 1]), hi);
              }
              w[j] = pack_bf16x2(lo * inv_scale, hi * inv_scale);
            }
            *reinterpret_cast<uint4*>(orow + cb * 32 + c8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      umma::fence_before_sync();
      mbar_arrive(B.o_free);
      // (d) Sb_{i+1} = bf16(St);  St <- g^C St
      if (i + 1 < nchunk) {
        ok = mbar_wait_abortable(B.st_ready, ph, s_abort);
        if (!__all_sync(0xffffffffu, ok)) break;
        umma::fence_after_sync();
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          umma::tmem_ld32(lane_base + kColSt + cb * 32, v);
          umma::tmem_wait_ld();
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w[j] = pack_bf16x2(__uint_as_float(v[c8 * 8 + 2 * j]), __uint_as_float(v[c8 * 8 + 2 * j + 1]));
            *reinterpret_cast<uint4*>(sb_tile + umma::tile_chunk_offset(r, cb * 32 + c8 * 8)) =
                make_uint4(w[0], w[1], w[2], w[3]);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * g_chunk);
          umma::tmem_st32(lane_base + kColSt + cb * 32, v);
        }
        umma::tmem_wait_st();
        umma::fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive(B.sb_ready);
      }
    }
  }

  // Teardown: everyone meets, the last MMA4 is drained, TMEM goes back.
  __syncwarp();
  if (warp == 1 && lane == 0 && !*s_abort) {
    // the final commit (st_ready of the last chunk) covers every MMA issued
    mbar_wait_abortable(B.st_ready, (nchunk - 1) & 1, s_abort);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  if (tid == 0 && *s_abort && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT);
  if (warp == 1) {
    __syncwarp();
    umma::tmem_dealloc(tmem, 512);
  }
}

}  // namespace

bool decayed_tc_supported(int B, int H, int T, int dk, int dv, int C, int dtype) {
  // TMA row coordinates are 32-bit signed
  return dtype == CB2_BF16 && dk == kC && dv == kC && C == kC && T % kC == 0 && T >= kC &&
         int64_t(B) * H * T < (int64_t(1) << 31);
}

int decayed_tc_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B,
                   int H, int T, int dk, int dv, int C, float scale, int* dev_status, cudaStream_t st) {
  (void)dk; (void)dv; (void)C;
  const uint64_t rows = uint64_t(B) * H * T;
  CUtensorMap mq, mk, mv;
  int rc = umma::make_tile_map(&mq, q, rows, kC);
  if (rc == CB2_OK) rc = umma::make_tile_map(&mk, k, rows, kC);
  if (rc == CB2_OK) rc = umma::make_tile_map(&mv, v, rows, kC);
  if (rc != CB2_OK) return rc;
  // per device, so set on every call (cheap) rather than cached per process
  if (cudaFuncSetAttribute(decayed_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           int(kSmemBytes)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  decayed_tc_kernel<<<B * H, kThreads, kSmemBytes, st>>>(mq, mk, mv, static_cast<__nv_bfloat16*>(o),
                                                        gamma, H, T, 1.0f / scale, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
