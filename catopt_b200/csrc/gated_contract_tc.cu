// Gated contraction  o = (s . g) @ v  on the 5th-generation tensor cores
// (bf16 tensors): the body of the reference's `om_decayed` element,
// `(s * d) @ v` (catopt_carriers/om.py:1053-1057), for a score tensor that is
// already materialised — the site the reference's generated-kernel tier lowers
// (`decayed_triton_bindings`, catopt_discovery/genkernel.py:1903-1925).  The
// gate g is any tensor of the scores' trailing shape (a decay mask, a causal
// mask, ...), shared over batch, per head, or per batch.
//
//   s: [nb, T, K]   g: [ng, T, K]   v: [nb, K, dv]   o: [nb, T, dv]
//   gate of batch b = g[(b / g_div) % g_mod]
//
// HBM-bound by its algorithmic bytes (s is read once: 2 bytes per 2*dv flops), but a
// 128-row CTA pulls three bytes through the L2 fabric for every score byte (scores,
// gate, and the values every row tile of a batch re-reads): about 12.6 TB/s from L2
// to the SMs at the measured pace of 0.5 us per stage, which deeper rings, a product
// kept out of shared memory and overlapped multiply groups all left unchanged.
// Scores and gate arrive by TMA (16 KiB
// each per 64-key stage; the gate usually from L2), a thread reads its row of both,
// and P = bf16(s . g) — rounded as the reference's elementwise multiply rounds it —
// is written to TENSOR MEMORY and is the A operand of O += P V_j from there; only V_j
// (MN-major B operand) is read from shared memory by the MMA.  fp32 accumulator in
// tensor memory.
//
// CTA = one 128-row tile of one batch; keys stream in 64-column stages (scores
// 16 KiB + gate 16 KiB + values 16 KiB) through a 2-slot ring, and two CTAs share an
// SM (97 KiB of shared memory and 256 TMEM columns each), so one CTA's ring fill and
// output store run under the other's steady state (measured: 4 slots x 1 CTA 247 us,
// 2 slots x 2 CTAs 238 us, 3 slots x 1 CTA 272 us on B=2 H=16 T=K=4096).
// Roles: warp 0 = TMA producer,
// warp 1 = MMA issuer and TMEM owner, warps 2..9 = multiply / epilogue group
// (thread = one row and one half of a stage's keys).  Rows past T and keys past K
// are out of range of the per-batch tensor maps: zero on load, clipped on store.
#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kRows = 128;                    // query rows per CTA
constexpr int kKeys = 64;                     // keys per stage
constexpr int kStages = 2;                    // ring slots per CTA
constexpr int kCtasPerSm = 2;
constexpr int kGcThreads = 320;
constexpr int kGcCompute = 256;
constexpr uint32_t kSBytes = kRows * kKeys * 2;          // 16 KiB score sub-tile
constexpr uint32_t kVHalf = kKeys * 128;                 // 8 KiB: 64 keys x 64 value columns
constexpr uint32_t kStageBytes = 2 * kSBytes + 2 * kVHalf;   // 48 KiB: scores, gate, values
constexpr uint32_t kGcOffOut = 0;    // output staging [128 x 128] bf16: over slot 0 of the ring, idle by then
constexpr uint32_t kGcOffBars = kStages * kStageBytes;
constexpr int kGcNumBars = 3 * kStages + 2;
constexpr uint32_t kGcOffMisc = kGcOffBars + kGcNumBars * 8;
constexpr uint32_t kGcSmemBytes = kGcOffMisc + 16 + 1024;
// tensor memory: accumulator in columns 0..127, then one 32-column P buffer per slot
// (64 keys of bf16, two per 32-bit column)
constexpr uint32_t kColP = 128;
constexpr uint32_t kGcTmemCols = 256;

__global__ void __launch_bounds__(kGcThreads, kCtasPerSm)
gated_contract_tc_kernel(const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_g,
                         const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                         int K, int dv, int row_tiles, int g_div, int g_mod, int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kGcOffBars);
  uint64_t* full = bars;                    // [kStages] TMA -> compute group, MMA
  uint64_t* p_ready = bars + kStages;       // [kStages] compute group -> MMA (256 arrivals)
  uint64_t* empty = bars + 2 * kStages;     // [kStages] MMA -> TMA
  uint64_t* acc_ready = bars + 3 * kStages; // last MMA done
  uint64_t* wg_sync = bars + 3 * kStages + 1;  // barrier among the 256 compute threads
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kGcOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kGcOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x / row_tiles;
  const int row0 = (blockIdx.x % row_tiles) * kRows;
  const int gb = (b / g_div) % g_mod;
  const int nstage = (K + kKeys - 1) / kKeys;
  const bool wide = dv > 64;                // second 64 value columns present

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&p_ready[s], kGcCompute);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
    mbar_init(wg_sync, kGcCompute);
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    umma::tmem_alloc(s_tmem, kGcTmemCols);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  if (warp == 0) {
    if (lane == 0) {
      umma::tma_prefetch_desc(&map_s);
      umma::tma_prefetch_desc(&map_g);
      umma::tma_prefetch_desc(&map_v);
      umma::tma_prefetch_desc(&map_o);
      const uint32_t bytes = 2 * kSBytes + (wide ? 2 : 1) * kVHalf;
      for (int i = 0; i < nstage; ++i) {
        const int slot = i % kStages, use = i / kStages;
        if (use > 0 && !mbar_wait_abortable(&empty[slot], (use - 1) & 1, s_abort)) break;
        unsigned char* dst = smem + slot * kStageBytes;
        const int k0 = i * kKeys;
        mbar_arrive_expect_tx(&full[slot], bytes);
        umma::tma_load_3d(dst, &map_s, k0, row0, b, &full[slot]);
        umma::tma_load_3d(dst + kSBytes, &map_g, k0, row0, gb, &full[slot]);
        umma::tma_load_3d(dst + 2 * kSBytes, &map_v, 0, k0, b, &full[slot]);
        if (wide) umma::tma_load_3d(dst + 2 * kSBytes + kVHalf, &map_v, 64, k0, b, &full[slot]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_wide = umma::instr_desc_bf16(128, 128, false, true);
      constexpr uint32_t idesc_narrow = umma::instr_desc_bf16(128, 64, false, true);
      const uint32_t idesc = wide ? idesc_wide : idesc_narrow;
      const uint32_t ring = smem_u32(smem);
      bool ok = true;
      for (int i = 0; i < nstage && ok; ++i) {
        const int slot = i % kStages, use = i / kStages;
        ok = mbar_wait_abortable(&full[slot], use & 1, s_abort) &&      // V_j landed
             mbar_wait_abortable(&p_ready[slot], use & 1, s_abort);     // P_j in tensor memory
        if (!ok) break;
        umma::fence_after_sync();
        const uint32_t v_addr = ring + slot * kStageBytes + 2 * kSBytes;
        const uint32_t p_addr = tmem + kColP + slot * 32;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          // A: tensor memory, 8 columns per 16-key step.
          // B: MN-major, 16 keys = 2048 B per k-step, 8-key groups 1024 B apart,
          //    value columns 64..127 in the second 8 KiB half.
          const uint64_t bdesc = umma::smem_desc(v_addr + ks * 2048u, kVHalf, 1024u);
          umma::mma_bf16_ts(tmem, p_addr + ks * 8, bdesc, idesc, i > 0 || ks > 0);
        }
        umma::mma_commit(&empty[slot]);
      }
      if (ok) umma::mma_commit(acc_ready);
    }
  } else {
    // thread = (row r of the tile, half of a stage's 64 keys); a warp may only touch
    // the TMEM lane quarter (warp % 4)
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q4 * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
    for (int i = 0; i < nstage; ++i) {
      const int slot = i % kStages, use = i / kStages;
      bool ok = mbar_wait_abortable(&full[slot], use & 1, s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      // P = bf16(s * g) for this thread's 32 keys of row r -> 16 packed columns of TMEM
      // (scores and gate share one swizzled layout; rows of a warp hit distinct banks)
      const unsigned char* s_tile = smem + slot * kStageBytes;
      uint4 xs[4], ys[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t off = umma::tile_chunk_offset(r, half * 32 + j * 8);
        xs[j] = *reinterpret_cast<const uint4*>(s_tile + off);
        ys[j] = *reinterpret_cast<const uint4*>(s_tile + kSBytes + off);
      }
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 x = xs[j];
        __nv_bfloat162* xa = reinterpret_cast<__nv_bfloat162*>(&x);
        const __nv_bfloat162* ya = reinterpret_cast<const __nv_bfloat162*>(&ys[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) xa[e] = __hmul2(xa[e], ya[e]);
        w[4 * j] = x.x; w[4 * j + 1] = x.y; w[4 * j + 2] = x.z; w[4 * j + 3] = x.w;
      }
      umma::tmem_st16(lane_base + kColP + slot * 32 + half * 16, w);
      umma::tmem_wait_st();
      umma::fence_before_sync();
      mbar_arrive(&p_ready[slot]);
    }
    // epilogue: thread = (row, column half); accumulator -> bf16 -> staged tile -> TMA store
    bool ok = mbar_wait_abortable(acc_ready, 0, s_abort);
    if (__all_sync(0xffffffffu, ok)) {
      umma::fence_after_sync();
      unsigned char* o_tile = smem + kGcOffOut;
      if (half == 0 || wide) {
        uint32_t va[32], vb[32];
        umma::tmem_ld32(lane_base + half * 64, va);
        umma::tmem_ld32(lane_base + half * 64 + 32, vb);
        umma::tmem_wait_ld();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(va[8 * c8]), __uint_as_float(va[8 * c8 + 1]));
          w.y = pack_bf16x2(__uint_as_float(va[8 * c8 + 2]), __uint_as_float(va[8 * c8 + 3]));
          w.z = pack_bf16x2(__uint_as_float(va[8 * c8 + 4]), __uint_as_float(va[8 * c8 + 5]));
          w.w = pack_bf16x2(__uint_as_float(va[8 * c8 + 6]), __uint_as_float(va[8 * c8 + 7]));
          *reinterpret_cast<uint4*>(o_tile + umma::tile_chunk_offset(r, half * 64 + c8 * 8)) = w;
          w.x = pack_bf16x2(__uint_as_float(vb[8 * c8]), __uint_as_float(vb[8 * c8 + 1]));
          w.y = pack_bf16x2(__uint_as_float(vb[8 * c8 + 2]), __uint_as_float(vb[8 * c8 + 3]));
          w.z = pack_bf16x2(__uint_as_float(vb[8 * c8 + 4]), __uint_as_float(vb[8 * c8 + 5]));
          w.w = pack_bf16x2(__uint_as_float(vb[8 * c8 + 6]), __uint_as_float(vb[8 * c8 + 7]));
          *reinterpret_cast<uint4*>(o_tile + umma::tile_chunk_offset(r, half * 64 + 32 + c8 * 8)) = w;
        }
      }
      umma::fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(wg_sync);
      ok = mbar_wait_abortable(wg_sync, 0, s_abort);   // whole tile staged (bounded like every wait)
      if (ok && tid == 64) {
        umma::tma_store_3d(&map_o, 0, row0, b, o_tile);
        if (wide) umma::tma_store_3d(&map_o, 64, row0, b, o_tile + umma::kSubTileBytes);
        bulk_commit();
        bulk_wait_all<0>();
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
    umma::tmem_dealloc(tmem, kGcTmemCols);
  }
}

}  // namespace

bool gated_contract_tc_supported(long long nb, int T, int K, int dv, int dtype, const void* s,
                                 const void* g, const void* v, const void* o) {
  return dtype == CB2_BF16 && K % 8 == 0 && dv % 8 == 0 && dv >= 8 && dv <= 128 && T >= 1 && K >= 1 &&
         T < (1 << 30) && K < (1 << 30) && nb * ((T + kRows - 1) / kRows) < (1ll << 31) && aligned16(s) &&
         aligned16(g) && aligned16(v) && aligned16(o);
}

int gated_contract_tc_run(const void* s, const void* g, const void* v, void* o, long long nb, long long ng,
                          int T, int K, int dv, int g_div, int g_mod, int* dev_status, cudaStream_t st) {
  CUtensorMap ms, mg, mv, mo;
  int rc = umma::make_map_3d(&ms, s, true, K, T, nb, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mg, g, true, K, T, ng, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mv, v, true, dv, K, nb, 64, 64, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mo, o, true, dv, T, nb, 64, 128, true);
  if (rc != CB2_OK) return rc;
  if (cudaFuncSetAttribute(gated_contract_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           int(kGcSmemBytes)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  const int row_tiles = (T + kRows - 1) / kRows;
  gated_contract_tc_kernel<<<unsigned(nb * row_tiles), kGcThreads, kGcSmemBytes, st>>>(
      ms, mg, mv, mo, K, dv, row_tiles, g_div, g_mod, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
