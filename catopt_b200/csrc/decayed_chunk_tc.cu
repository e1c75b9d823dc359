// Chunked decayed attention on the 5th-generation tensor cores (bf16 tensors,
// dk, dv <= 128, any T): one CTA per (batch, head) walks 128-row
// chunks in order and keeps the fp32 inter-chunk state in tensor memory for the
// whole sequence.  The value does not depend on the chunking, so the kernel
// always uses 128-row chunks whatever chunk size the lowered term was cut into;
// head dimensions below 128 and a ragged last chunk are zero-padded for free by
// the TMA (columns past dk / dv and rows past T are out of range of the per-head
// tensor map: they arrive as zeros, contribute nothing, and are clipped on store).
//
// Per chunk i (C = 128 rows, g = gamma of the head):
//   MMA1  S  = Q_i K_i^T                                  (TMEM cols   0..127)
//   WG    P  = bf16( S . tril(g^(r-c)) )  -> TMEM (over S) ;  K_i <- K_i . g^(C-1-r) in place
//   MMA2  O1 = P V_i        (A operand read from TMEM)      (TMEM cols 128..255)
//   MMA3  O2 = Q_i Sb_i        (Sb_i = bf16 copy of the state, i > 0)   (256..383)
//   WG    o_i = (O1 + g^(r+1) O2) / scale  -> staged in shared memory, TMA store
//   MMA4  St = [g^C St] + Kw_i^T V_i                       (TMEM cols 384..511)
//   WG    (during the next chunk's MMA2)  Sb_{i+1} = bf16(St) -> smem ;  St <- g^C St
// which is the state-carry recurrence the reference spells in
// lab/probes/retnet_baseline_probe.py:77-110 and equals its pairwise executor
// (decayed_lower.py:671-700) up to reassociation.  Only chunk-local powers of g
// appear.
//
// Heads are equal-sized, so B*H CTAs on 148 SMs leave the last wave partly
// empty (512 heads: 3.46 waves cost 4).  When the caller provides scratch, each
// head is therefore cut into n_seg consecutive segments of chunks, one CTA
// each, launched segment-major: segment s of a head takes the fp32 state that
// segment s-1 left in scratch (64 KiB) once a flag says it is there.  A CTA's
// predecessor has a lower block index, so it is running or finished whenever
// the CTA itself runs; the wait is bounded like every other.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer (and TMEM owner),
// warps 2..9 = the 256-thread compute group (thread = one TMEM lane = one row,
// half of the columns).
// Operand tiles (32 KiB each, K_i / Q_i / V_i in that order) stream through a
// shared-memory ring with full/empty mbarriers; a slot is released by the
// tcgen05.commit of the last MMA that reads it.  The common-case roles use six
// slots — two whole chunks, so the loads of chunk i+1 are issued about a chunk
// ahead of their use (a tile lands 2-3 k cycles after its request; with less
// lookahead the chunk time is that latency, not the work) — and stage o_i over
// the chunk's own Q tile once MMA1 and MMA3 have read it; the every-rate roles
// keep five slots and a separate staging tile.  HBM traffic is exactly the
// algorithmic bytes: q, k, v read once, o written once.
#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kC = 128;                 // chunk rows = dk = dv
constexpr unsigned long long kWaitNs = kDefaultWaitNs;   // budget of every wait; a wait that runs out reports its source line
constexpr int kSlots = 5;                     // ring depth of the every-rate roles
constexpr int kSlotsFast = 6;                 // ring depth of the common-case roles (two whole chunks)
constexpr int kSlotsMax = 6;
constexpr int kThreads = 320;                 // 2 single-lane role warps + 8 compute warps
constexpr int kComputeThreads = 256;
constexpr uint32_t kTile = umma::kTileBytes;      // 32 KiB
// shared memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffRing = 0;
constexpr uint32_t kOffO = kSlots * kTile;          // output staging tile of the every-rate roles (= the sixth ring tile)
constexpr uint32_t kOffSb = kSlotsMax * kTile;
constexpr uint32_t kOffPow = kOffSb + kTile;                 // float[32 zeros | g^0 .. g^128]
constexpr uint32_t kOffBars = kOffPow + 704;                 // 8-byte aligned
constexpr int kNumBars = 2 * kSlotsMax + 9;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;       // tmem base, abort flag
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;        // + alignment slack

// TMEM columns
constexpr uint32_t kColS = 0, kColO1 = 128, kColO2 = 256, kColSt = 384;
// P (bf16, two values per 32-bit column) overwrites S in place: the thread that
// read S columns [64h, 64h+64) writes the packed P of those columns into
// [64h, 64h+32), i.e. only over columns it has already loaded itself.
__host__ __device__ constexpr uint32_t p_col(uint32_t c) { return (c & 64u) + ((c & 63u) >> 1); }

struct Bars {
  uint64_t* full;      // [kSlotsMax] TMA -> MMA
  uint64_t* empty;     // [kSlotsMax] MMA -> TMA
  uint64_t* s_ready;   // MMA1 done            (MMA -> WG)
  uint64_t* p_ready;   // P written            (WG -> MMA, 256 arrivals)
  uint64_t* kw_ready;  // K scaled in place    (WG -> MMA, 256)
  uint64_t* o_ready;   // MMA2+MMA3 done       (MMA -> WG)
  uint64_t* o_free;    // O1/O2 read out       (WG -> MMA, 256)
  uint64_t* st_ready;  // MMA4 done            (MMA -> WG)
  uint64_t* sb_ready;  // Sb written, St scaled (WG -> MMA, 256)
  uint64_t* wg_sync;   // barrier among the 256 compute threads
  uint64_t* kw_taken;  // the MMA thread has seen kw_ready of a chunk (MMA -> WG)
};


// The state a later segment starts from (this thread's 64 elements of row r: columns cb0*32 ..
// +63), ready before the launch.  pieces_per_seg == 0: the finished start state sits in slot
// seg-1 (written by the scan kernel of decayed_seg_state.cu).  Otherwise the slots hold the end
// states E_p (from zero) of consecutive pieces of `piece_rows` rows, pieces_per_seg of them per
// segment, and the start state is their fold  S = g^(piece_rows) S + E_p  over the pieces before
// this segment (at most four: a fold in every CTA is then cheaper than one more launch).
__device__ __forceinline__ void load_start_state(const float* seg_state, int seg, int n_bh, int bh, int r, int cb0,
                                                 int pieces_per_seg, float g_piece, uint32_t (&va)[32],
                                                 uint32_t (&vb)[32]) {
  const size_t elem = size_t(r) * kC + cb0 * 32;
  if (pieces_per_seg == 0) {
    const float4* src = reinterpret_cast<const float4*>(seg_state + (size_t(seg - 1) * n_bh + bh) * (kC * kC) + elem);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 x = __ldcg(src + j), y = __ldcg(src + 8 + j);
      va[4 * j] = __float_as_uint(x.x); va[4 * j + 1] = __float_as_uint(x.y);
      va[4 * j + 2] = __float_as_uint(x.z); va[4 * j + 3] = __float_as_uint(x.w);
      vb[4 * j] = __float_as_uint(y.x); vb[4 * j + 1] = __float_as_uint(y.y);
      vb[4 * j + 2] = __float_as_uint(y.z); vb[4 * j + 3] = __float_as_uint(y.w);
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) va[j] = vb[j] = 0u;
  const int n = seg * pieces_per_seg;
  for (int p = 0; p < n; ++p) {
    const float4* src = reinterpret_cast<const float4*>(seg_state + (size_t(p) * n_bh + bh) * (kC * kC) + elem);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 x = __ldcg(src + j), y = __ldcg(src + 8 + j);
      va[4 * j] = __float_as_uint(fmaf(g_piece, __uint_as_float(va[4 * j]), x.x));
      va[4 * j + 1] = __float_as_uint(fmaf(g_piece, __uint_as_float(va[4 * j + 1]), x.y));
      va[4 * j + 2] = __float_as_uint(fmaf(g_piece, __uint_as_float(va[4 * j + 2]), x.z));
      va[4 * j + 3] = __float_as_uint(fmaf(g_piece, __uint_as_float(va[4 * j + 3]), x.w));
      vb[4 * j] = __float_as_uint(fmaf(g_piece, __uint_as_float(vb[4 * j]), y.x));
      vb[4 * j + 1] = __float_as_uint(fmaf(g_piece, __uint_as_float(vb[4 * j + 1]), y.y));
      vb[4 * j + 2] = __float_as_uint(fmaf(g_piece, __uint_as_float(vb[4 * j + 2]), y.z));
      vb[4 * j + 3] = __float_as_uint(fmaf(g_piece, __uint_as_float(vb[4 * j + 3]), y.w));
    }
  }
}

// ---------------------------------------------------------------------------------------
// Roles of the common case: decay rates close enough to one (g >= 0.74) that the powers
// g^(-c) of a whole chunk fit comfortably in bf16/fp32 range.  Writing the decay mask as
// g^(r-c) = g^r . g^(-c) moves every per-element multiply out of the compute group:
//
//   K~_i  = K_i . g^(-c - C.mi)          (row c of the tile scaled once, BEFORE MMA1; the same
//                                         tile feeds MMA1 and MMA4; mi = chunk index mod m)
//   MMA1  S' = Q_i K~_i^T
//   WG    P' = bf16(S') below the diagonal, 0 above      (a select, no table, no multiply)
//   MMA2  O' = P' V_i          MMA3  O' += Q_i Sb         (ONE accumulator: both terms carry
//   WG    o_i = g^(r + C.mi) / scale . O'  -> global       the same row factor)
//   MMA4  A += K~_i^T V_i      (the raw accumulator: true state = g^(C.mi' - 1) . A)
//   WG    Sb = bf16(A) for the next chunk; every m chunks A <- g^(C.m) A  (m = the largest
//         power of two with g^(-C.m) <= 2^56, so A never leaves fp32 range; m = 8 at g = 0.969)
//
// Per chunk the compute group now loads 192 and stores 32 TMEM words per thread (was 256 and
// 96) and multiplies 128 values (was 320); the state chain (MMA4 -> Sb -> MMA3) no longer
// passes through a rescale of the accumulator.  Issue order per chunk: MMA1, MMA4, MMA2, MMA3 —
// MMA4 needs nothing from the mask, so it fills the tensor core's wait for P'.
// The renormalisation points are multiples of m in the GLOBAL chunk index and a flagged
// hand-off passes the raw accumulator, so a head cut into segments that wait for one another
// gives the same bits as one CTA walking the head.
// Heads served by several CTAs of one launch without scratch: CTA j of a head produces chunks
// [s[j], s[j+1]) and first walks [0, s[j]) for the state only.  ways == 0: not used.
struct SelfSplit {
  int ways;
  int s[5];
};

struct FastCtx {
  unsigned char* smem;
  Bars B;
  uint32_t tmem;
  const CUtensorMap *map_q, *map_k, *map_v, *map_o;
  int bh, seg, n_bh, n_seg, nchunk, chunk0, dv, prestaged, pieces_per_seg;
  float g_piece;            // g^(rows of a precomputed piece)
  bool has_in;
  float lg, inv_scale;      // lg = -log2(g)
  float* seg_state;
  int* seg_flag;
  volatile int* s_abort;
  int pre;                  // leading chunks (an even count) walked for their state only
};

__device__ __forceinline__ void fast_roles(const FastCtx& c) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Bars& B = c.B;
  unsigned char* smem = c.smem;
  volatile int* s_abort = c.s_abort;
  const int nchunk = c.nchunk;
  const bool has_in = c.has_in;
  const int pre = c.pre;
  const uint32_t tmem = c.tmem;
  const uint32_t ring_addr = smem_u32(smem + kOffRing);
  const uint32_t sb_addr = smem_u32(smem + kOffSb);
  constexpr uint32_t kColO = kColO1, kColA = kColSt;
  // renormalisation period: the largest power of two m <= 64 with C.m.lg <= 56
  int m = 1;
  while (m < 64 && float(2 * m * kC) * c.lg <= 56.f) m *= 2;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      umma::tma_prefetch_desc(c.map_q);
      umma::tma_prefetch_desc(c.map_k);
      umma::tma_prefetch_desc(c.map_v);
      umma::tma_prefetch_desc(c.map_o);
      const int ntiles = 3 * nchunk;
      for (int t = 0; t < ntiles; ++t) {
        const int i = t / 3, which = t % 3;  // 0: K, 1: Q, 2: V
        if (which == 1 && i < pre) continue;       // state-only chunk: no Q
        // K and V slots are used by every chunk; the two Q slots only from chunk `pre` (even) on
        const int slot = t % kSlotsFast, use = which == 1 ? (i - pre) / 2 : t / kSlotsFast;
        if (use > 0 && !mbar_wait_abortable(&B.empty[slot], (use - 1) & 1, s_abort, kWaitNs, __LINE__)) break;
        const CUtensorMap* mp = which == 0 ? c.map_k : (which == 1 ? c.map_q : c.map_v);
        unsigned char* dst = smem + kOffRing + slot * kTile;
        const int row = (c.chunk0 + i) * kC;
        mbar_arrive_expect_tx(&B.full[slot], kTile);
        umma::tma_load_3d(dst, mp, 0, row, c.bh, &B.full[slot]);
        umma::tma_load_3d(dst + umma::kSubTileBytes, mp, 64, row, c.bh, &B.full[slot]);
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
        const uint32_t k_addr = ring_addr + (tk % kSlotsFast) * kTile;
        const uint32_t q_addr = ring_addr + (tq % kSlotsFast) * kTile;
        const uint32_t v_addr = ring_addr + (tv % kSlotsFast) * kTile;
        const bool state_only = i < pre;
        // MMA1: S' = Q K~^T  (K~ is ready once the compute group has scaled the tile)
        if (!mbar_wait_abortable(B.kw_ready, ph, s_abort, kWaitNs, __LINE__)) break;
        mbar_arrive(B.kw_taken);            // (see scale_k: the group may now signal the chunk after this one)
        if (!state_only) {
          if (!mbar_wait_abortable(&B.full[tq % kSlotsFast], ((i - pre) / 2) & 1, s_abort, kWaitNs, __LINE__)) break;
          umma::fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma::mma_bf16(tmem + kColS, umma::desc_kmajor(q_addr, ks), umma::desc_kmajor(k_addr, ks),
                           idesc_kk, ks > 0);
          umma::mma_commit(B.s_ready);
        }
        // MMA4: A (+)= K~^T V.  Issued ahead of MMA2/MMA3: it does not depend on the mask, so the
        // tensor core works through it while the compute group turns S' into P'.  The compute
        // group must have finished copying the previous accumulator into Sb first.
        if (!mbar_wait_abortable(&B.full[tv % kSlotsFast], (tv / kSlotsFast) & 1, s_abort, kWaitNs, __LINE__)) break;
        if (i > 0 || has_in) {
          if (!mbar_wait_abortable(B.sb_ready, (has_in ? i : i - 1) & 1, s_abort, kWaitNs, __LINE__)) break;
        }
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16(tmem + kColA, umma::desc_mnmajor(k_addr, ks), umma::desc_mnmajor(v_addr, ks),
                         idesc_nn, (i > 0) || has_in || (ks > 0));
        umma::mma_commit(&B.empty[tk % kSlotsFast]);
        if (state_only) {                 // nothing else in a state-only chunk
          umma::mma_commit(&B.empty[tv % kSlotsFast]);
          umma::mma_commit(B.o_ready);
          umma::mma_commit(B.st_ready);
          continue;
        }
        // MMA2: O' = P' V
        if (!mbar_wait_abortable(B.p_ready, ph, s_abort, kWaitNs, __LINE__)) break;
        if (i > pre && !mbar_wait_abortable(B.o_free, (i - 1) & 1, s_abort, kWaitNs, __LINE__)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16_ts(tmem + kColO, tmem + kColS + p_col(ks * 16),
                            umma::desc_mnmajor(v_addr, ks), idesc_kn, ks > 0);
        umma::mma_commit(&B.empty[tv % kSlotsFast]);
        // MMA3: O' += Q Sb  (no state before the first chunk of the sequence)
        if (i > 0 || has_in) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma::mma_bf16(tmem + kColO, umma::desc_kmajor(q_addr, ks),
                           umma::desc_mnmajor(sb_addr, ks), idesc_kn, true);
        }
        umma::mma_commit(B.o_ready);     // every MMA of the chunk is done (the Q slot is released by the
        umma::mma_commit(B.st_ready);    // compute group: it stages o_i there)
      }
    }
  } else {
    // ------------------------------------------------------------ compute group
    const int q4 = warp & 3;                 // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;        // 0: columns 0..63, 1: columns 64..127
    const int r = q4 * 32 + lane;            // row of the chunk / lane of TMEM
    const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
    unsigned char* sb_tile = smem + kOffSb;
    const float g_renorm = exp2f(-c.lg * float(m * kC));        // g^(C.m)
    uint32_t va[32], vb[32];
    uint32_t wg_phase = 0;
    auto store_block = [&](unsigned char* tile, int col0, const uint32_t (&w)[16]) {
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8)
        *reinterpret_cast<uint4*>(tile + umma::tile_chunk_offset(r, col0 + c8 * 8)) =
            make_uint4(w[4 * c8], w[4 * c8 + 1], w[4 * c8 + 2], w[4 * c8 + 3]);
    };
    // K~_j = K_j . g^(-r - C.mj), in place, as soon as the tile has landed
    auto scale_k = [&](int j) -> bool {
      const int tk = 3 * j;
      bool ok = mbar_wait_abortable(&B.full[tk % kSlotsFast], (tk / kSlotsFast) & 1, s_abort, kWaitNs, __LINE__);
      if (!__all_sync(0xffffffffu, ok)) return false;
      const float kf = exp2f(c.lg * float(r + kC * ((c.chunk0 + j) % m)));
      unsigned char* k_tile = smem + kOffRing + (tk % kSlotsFast) * kTile;
      uint4 x[8];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj)
        x[jj] = *reinterpret_cast<const uint4*>(k_tile + umma::tile_chunk_offset(r, half * 64 + jj * 8));
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        x[jj].x = pack_bf16x2(bf16lo_to_f32(x[jj].x) * kf, bf16hi_to_f32(x[jj].x) * kf);
        x[jj].y = pack_bf16x2(bf16lo_to_f32(x[jj].y) * kf, bf16hi_to_f32(x[jj].y) * kf);
        x[jj].z = pack_bf16x2(bf16lo_to_f32(x[jj].z) * kf, bf16hi_to_f32(x[jj].z) * kf);
        x[jj].w = pack_bf16x2(bf16lo_to_f32(x[jj].w) * kf, bf16hi_to_f32(x[jj].w) * kf);
      }
#pragma unroll
      for (int jj = 0; jj < 8; ++jj)
        *reinterpret_cast<uint4*>(k_tile + umma::tile_chunk_offset(r, half * 64 + jj * 8)) = x[jj];
      fence_proxy_async_smem();
      // One signal ahead of the MMA thread at most: a waiter on a phase parity cannot tell phase j - 1 from
      // phase j + 1, and in a state-only chunk nothing else keeps this group from signalling chunk j before
      // the MMA thread has looked at the signal of chunk j - 1 (it then waits for a phase that needs it to
      // move first, and every wait of the CTA runs out).  Happened with eight ranks on one node in the host
      // pipeline, never on one to four GPUs; holding the MMA thread back 40 us at its start makes it certain
      // without this wait and impossible with it.
      if (j > 0) {
        ok = mbar_wait_abortable(B.kw_taken, (j - 1) & 1, s_abort, kWaitNs, __LINE__);
        if (!__all_sync(0xffffffffu, ok)) return false;
      }
      mbar_arrive(B.kw_ready);
      return true;
    };
    bool alive = scale_k(0);
    for (int i = 0; alive && i < nchunk; ++i) {
      const uint32_t ph = i & 1;
      const int mi = (c.chunk0 + i) % m;
      const bool state_only = i < pre;
      bool ok = true;
      if (state_only) {
        // K and V only: the accumulator just grows (MMA4); every m chunks it is renormalised here.
        // (o_ready of the previous chunk, waited for below, says its MMA4 has completed.)
        if (i > 0) {
          if (mi == 0) {
            const int cb0 = half * 2;
            umma::tmem_ld32(lane_base + kColA + cb0 * 32, va);
            umma::tmem_ld32(lane_base + kColA + cb0 * 32 + 32, vb);
            umma::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              va[j] = __float_as_uint(__uint_as_float(va[j]) * g_renorm);
              vb[j] = __float_as_uint(__uint_as_float(vb[j]) * g_renorm);
            }
            umma::tmem_st32(lane_base + kColA + cb0 * 32, va);
            umma::tmem_st32(lane_base + kColA + cb0 * 32 + 32, vb);
            umma::tmem_wait_st();
          }
          umma::fence_before_sync();
          mbar_arrive(B.sb_ready);
        }
        if (i + 1 < nchunk && !scale_k(i + 1)) break;
        ok = mbar_wait_abortable(B.o_ready, ph, s_abort, kWaitNs, __LINE__);
        if (!__all_sync(0xffffffffu, ok)) break;
        umma::fence_after_sync();
        continue;
      }
      // (s) Sb = bf16(A) for this chunk's MMA3.  First thing in the iteration: the accumulator is
      // final and Sb is free once every MMA of the previous chunk has completed, and the copy then
      // runs under MMA1 of this chunk (operands from shared memory: the tensor-memory read port is
      // free); MMA4 of this chunk waits for it
      if (i > 0 || has_in) {
        const int cb0 = half * 2;
        float mult = 1.f;
        bool writeback = false;
        if (i > 0) {
          // (o_ready of the previous chunk, which this thread has waited for, covers its MMA3 and MMA4)
          umma::tmem_ld32(lane_base + kColA + cb0 * 32, va);
          umma::tmem_ld32(lane_base + kColA + cb0 * 32 + 32, vb);
          umma::tmem_wait_ld();
          if (mi == 0) { mult = g_renorm; writeback = true; }
        } else {
          // first chunk of a later segment: prestaged = the true state before this chunk,
          // computed ahead of the launch; otherwise the predecessor CTA's raw accumulator
          if (!c.prestaged) {
            const int* flag = c.seg_flag + size_t(c.seg - 1) * c.n_bh + c.bh;
            ok = wait_flag_abortable(flag, s_abort, kWaitNs, __LINE__);
            if (!__all_sync(0xffffffffu, ok)) break;
          }
          load_start_state(c.seg_state, c.seg, c.n_bh, c.bh, r, cb0, c.prestaged ? c.pieces_per_seg : 0, c.g_piece,
                           va, vb);
          writeback = true;
          mult = c.prestaged ? exp2f(c.lg * float(kC * mi - 1)) : (mi == 0 ? g_renorm : 1.f);
        }
        if (mult != 1.f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            va[j] = __float_as_uint(__uint_as_float(va[j]) * mult);
            vb[j] = __float_as_uint(__uint_as_float(vb[j]) * mult);
          }
        }
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          w[j >> 1] = pack_bf16x2(__uint_as_float(va[j]), __uint_as_float(va[j + 1]));
        store_block(sb_tile, cb0 * 32, w);
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          w[j >> 1] = pack_bf16x2(__uint_as_float(vb[j]), __uint_as_float(vb[j + 1]));
        store_block(sb_tile, cb0 * 32 + 32, w);
        if (writeback) {
          umma::tmem_st32(lane_base + kColA + cb0 * 32, va);
          umma::tmem_st32(lane_base + kColA + cb0 * 32 + 32, vb);
          umma::tmem_wait_st();
        }
        umma::fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive(B.sb_ready);
      }
      ok = mbar_wait_abortable(B.s_ready, ph, s_abort, kWaitNs, __LINE__);
      if (!__all_sync(0xffffffffu, ok)) break;
      umma::fence_after_sync();
      // (a) P' = bf16(S') at and below the diagonal, 0 above, packed into TMEM over S'
      {
        const int cb0 = half * 2, cb1 = cb0 + 1;
        if (cb0 <= q4) umma::tmem_ld32(lane_base + kColS + cb0 * 32, va);
        if (cb1 <= q4) umma::tmem_ld32(lane_base + kColS + cb1 * 32, vb);
        if (cb0 <= q4) umma::tmem_wait_ld();
        auto mask_block = [&](int cb, const uint32_t (&v)[32]) {
          uint32_t w[16];
          if (cb < q4) {
#pragma unroll
            for (int j = 0; j < 32; j += 2)
              w[j >> 1] = pack_bf16x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
          } else if (cb == q4) {
#pragma unroll
            for (int j = 0; j < 32; j += 2)
              w[j >> 1] = pack_bf16x2(j <= lane ? __uint_as_float(v[j]) : 0.f,
                                      j + 1 <= lane ? __uint_as_float(v[j + 1]) : 0.f);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = 0u;
          }
          umma::tmem_st16(lane_base + kColS + p_col(cb * 32), w);
        };
        mask_block(cb0, va);
        mask_block(cb1, vb);
        umma::tmem_wait_st();
      }
      umma::fence_before_sync();
      mbar_arrive(B.p_ready);
      // the previous chunk's output has left the ring tile it was staged in (that chunk's Q
      // tile): hand the slot back to the producer
      if (tid == 64 && i > pre) {
        bulk_wait_read<0>();
        mbar_arrive(&B.empty[(3 * (i - 1) + 1) % kSlotsFast]);
      }
      // (k) the next chunk's K tile, scaled ahead of its MMA1
      if (i + 1 < nchunk && !scale_k(i + 1)) break;
      // (c) o_i = g^(r + C.mi) / scale . O'
      ok = mbar_wait_abortable(B.o_ready, ph, s_abort, kWaitNs, __LINE__);
      if (!__all_sync(0xffffffffu, ok)) break;
      umma::fence_after_sync();
      // staged in the chunk's own Q tile (MMA1 and MMA3 are done with it) in the swizzled layout the
      // TMA store expects.  (Storing straight from registers — every thread owns 128 contiguous
      // bytes of its row — was measured at 3 k cycles per chunk for this phase: 32 rows a warp,
      // 256 bytes apart, is the worst case for the store path.)
      unsigned char* o_tile = smem + kOffRing + ((3 * i + 1) % kSlotsFast) * kTile;
      {
        const float f = exp2f(-c.lg * float(r + kC * mi)) * c.inv_scale;
        const int cb0 = half * 2;
        umma::tmem_ld32(lane_base + kColO + cb0 * 32, va);
        umma::tmem_ld32(lane_base + kColO + cb0 * 32 + 32, vb);
        umma::tmem_wait_ld();
        umma::fence_before_sync();
        mbar_arrive(B.o_free);                 // O' is in registers: MMA2 of the next chunk may start
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          w[j >> 1] = pack_bf16x2(__uint_as_float(va[j]) * f, __uint_as_float(va[j + 1]) * f);
        store_block(o_tile, cb0 * 32, w);
#pragma unroll
        for (int j = 0; j < 32; j += 2)
          w[j >> 1] = pack_bf16x2(__uint_as_float(vb[j]) * f, __uint_as_float(vb[j + 1]) * f);
        store_block(o_tile, cb0 * 32 + 32, w);
      }
      fence_proxy_async_smem();
      mbar_arrive(B.wg_sync);
      ok = mbar_wait_abortable(B.wg_sync, wg_phase, s_abort, kWaitNs, __LINE__);
      wg_phase ^= 1;
      if (!__all_sync(0xffffffffu, ok)) break;
      if (tid == 64) {
        const int row = (c.chunk0 + i) * kC;   // the store is clipped at T
        umma::tma_store_3d(c.map_o, 0, row, c.bh, o_tile);
        if (c.dv > 64) umma::tma_store_3d(c.map_o, 64, row, c.bh, o_tile + umma::kSubTileBytes);
        bulk_commit();
      }
    }
    // hand the raw accumulator to the next segment of this head
    if (c.seg + 1 < c.n_seg && !c.prestaged) {
      bool ok = mbar_wait_abortable(B.st_ready, (nchunk - 1) & 1, s_abort, kWaitNs, __LINE__);
      if (__all_sync(0xffffffffu, ok)) {
        umma::fence_after_sync();
        const int cb0 = half * 2;
        umma::tmem_ld32(lane_base + kColA + cb0 * 32, va);
        umma::tmem_ld32(lane_base + kColA + cb0 * 32 + 32, vb);
        umma::tmem_wait_ld();
        float4* dst = reinterpret_cast<float4*>(c.seg_state + (size_t(c.seg) * c.n_bh + c.bh) * (kC * kC) +
                                                r * kC + cb0 * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __stcg(dst + j, make_float4(__uint_as_float(va[4 * j]), __uint_as_float(va[4 * j + 1]),
                                      __uint_as_float(va[4 * j + 2]), __uint_as_float(va[4 * j + 3])));
          __stcg(dst + 8 + j, make_float4(__uint_as_float(vb[4 * j]), __uint_as_float(vb[4 * j + 1]),
                                          __uint_as_float(vb[4 * j + 2]), __uint_as_float(vb[4 * j + 3])));
        }
        __threadfence();
        mbar_arrive(B.wg_sync);
        ok = mbar_wait_abortable(B.wg_sync, wg_phase, s_abort, kWaitNs, __LINE__);
        wg_phase ^= 1;
        if (ok && tid == 64) {
          int* flag = c.seg_flag + size_t(c.seg) * c.n_bh + c.bh;
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
        }
      }
    }
    if (tid == 64) bulk_wait_all<0>();  // the staged output has left shared memory
  }
}

__global__ void __launch_bounds__(kThreads, 1)
decayed_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                  const float* __restrict__ gamma, int H, int T, int dv, float inv_scale, int n_bh, int n_seg,
                  float* __restrict__ seg_state, int* __restrict__ seg_flag, int prestaged, int pieces_per_seg,
                  int piece_rows, const SelfSplit self, int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles; plain offset arithmetic on the
  // __shared__ array keeps every access a shared-space (LDS/STS) access
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // s_pow[j] = g^j for j in [-32, 128]; negative exponents hold 0, so the causal
  // mask of the diagonal block needs neither a clamp nor a select
  float* s_pow = reinterpret_cast<float*>(smem + kOffPow) + 32;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 4);
  Bars B{bars, bars + kSlotsMax, bars + 2 * kSlotsMax, bars + 2 * kSlotsMax + 1, bars + 2 * kSlotsMax + 2,
         bars + 2 * kSlotsMax + 3, bars + 2 * kSlotsMax + 4, bars + 2 * kSlotsMax + 5, bars + 2 * kSlotsMax + 6,
         bars + 2 * kSlotsMax + 7, bars + 2 * kSlotsMax + 8};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x % n_bh;
  const int seg = blockIdx.x / n_bh;               // segment-major launch order
  const float g = gamma[bh % H];
  // decay rates in [0.74, 1]: the cheaper formulation (see fast_roles); anything else keeps
  // the chunk-local decaying powers, which are safe for every rate
  const float lg = -log2f(g);
  const bool fast = g > 0.f && g <= 1.f && float(kC) * lg <= 56.f;
  int nchunk = (T + kC - 1) / kC / n_seg;          // chunks of this segment
  int chunk0 = seg * nchunk;                       // first chunk of the segment in the sequence
  bool has_in = seg > 0;                           // starts from a predecessor's state
  int pre = 0;                                     // leading chunks walked for their state only
  if (self.ways > 0) {
    // Several CTAs per head, no scratch, no flags, one launch: CTA j walks chunks [0, s[j]) only to
    // accumulate their state (K and V alone, no scores, no output) and produces [s[j], s[j+1]).
    // (n_seg == 1 here.)
    chunk0 = 0;
    has_in = false;
    if (fast) {
      pre = self.s[seg];
      nchunk = self.s[seg + 1];
    } else if (seg != 0) {
      nchunk = 0;                                  // the every-rate roles walk the head in one CTA
    }
  }
  const uint32_t ring_addr = smem_u32(smem + kOffRing);
  const uint32_t sb_addr = smem_u32(smem + kOffSb);

  if (tid == 0) {
    for (int s = 0; s < kSlotsMax; ++s) {
      mbar_init(&B.full[s], 1);
      mbar_init(&B.empty[s], 1);
    }
    mbar_init(B.s_ready, 1);
    mbar_init(B.p_ready, kComputeThreads);
    mbar_init(B.kw_ready, kComputeThreads);
    mbar_init(B.o_ready, 1);
    mbar_init(B.o_free, kComputeThreads);
    mbar_init(B.st_ready, 1);
    mbar_init(B.sb_ready, kComputeThreads);
    mbar_init(B.wg_sync, kComputeThreads);
    mbar_init(B.kw_taken, 1);
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    umma::tmem_alloc(s_tmem, 512);
  }
  if (tid >= 64 && tid < 192) {  // powers of gamma for this head: g^0 .. g^128
    const int j = tid - 64;
    s_pow[j] = powf(g, float(j));
    if (j == 0) s_pow[kC] = powf(g, float(kC));
    if (j < 32) s_pow[j - 32] = 0.f;
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  if (fast) {
    fast_roles(FastCtx{smem, B, tmem, &map_q, &map_k, &map_v, &map_o, bh, seg, n_bh, n_seg, nchunk, chunk0, dv,
                       prestaged, pieces_per_seg, exp2f(-lg * float(piece_rows)), has_in, lg, inv_scale, seg_state,
                       seg_flag, s_abort, pre});
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      umma::tma_prefetch_desc(&map_q);
      umma::tma_prefetch_desc(&map_k);
      umma::tma_prefetch_desc(&map_v);
      umma::tma_prefetch_desc(&map_o);
      const int ntiles = 3 * nchunk;
      for (int t = 0; t < ntiles; ++t) {
        const int slot = t % kSlots, use = t / kSlots;
        if (use > 0 && !mbar_wait_abortable(&B.empty[slot], (use - 1) & 1, s_abort, kWaitNs, __LINE__)) break;
        const int i = t / 3, which = t % 3;  // 0: K, 1: Q, 2: V
        const CUtensorMap* m = which == 0 ? &map_k : (which == 1 ? &map_q : &map_v);
        unsigned char* dst = smem + kOffRing + slot * kTile;
        const int row = (chunk0 + i) * kC;   // rows past T (ragged last chunk) arrive as zeros
        mbar_arrive_expect_tx(&B.full[slot], kTile);
        umma::tma_load_3d(dst, m, 0, row, bh, &B.full[slot]);
        umma::tma_load_3d(dst + umma::kSubTileBytes, m, 64, row, bh, &B.full[slot]);
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
        if (!mbar_wait_abortable(&B.full[tk % kSlots], (tk / kSlots) & 1, s_abort, kWaitNs, __LINE__)) break;
        if (!mbar_wait_abortable(&B.full[tq % kSlots], (tq / kSlots) & 1, s_abort, kWaitNs, __LINE__)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16(tmem + kColS, umma::desc_kmajor(q_addr, ks), umma::desc_kmajor(k_addr, ks),
                         idesc_kk, ks > 0);
        umma::mma_commit(B.s_ready);
        // MMA2: O1 = P V
        if (!mbar_wait_abortable(B.p_ready, ph, s_abort, kWaitNs, __LINE__)) break;
        if (!mbar_wait_abortable(&B.full[tv % kSlots], (tv / kSlots) & 1, s_abort, kWaitNs, __LINE__)) break;
        if (i > 0 && !mbar_wait_abortable(B.o_free, (i - 1) & 1, s_abort, kWaitNs, __LINE__)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16_ts(tmem + kColO1, tmem + kColS + p_col(ks * 16),
                            umma::desc_mnmajor(v_addr, ks), idesc_kn, ks > 0);
        // MMA3: O2 = Q Sb   (the state is zero before the first chunk of the sequence)
        if (i > 0 || has_in) {
          if (!mbar_wait_abortable(B.sb_ready, (has_in ? i : i - 1) & 1, s_abort, kWaitNs, __LINE__)) break;
          umma::fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma::mma_bf16(tmem + kColO2, umma::desc_kmajor(q_addr, ks),
                           umma::desc_mnmajor(sb_addr, ks), idesc_kn, ks > 0);
        }
        umma::mma_commit(B.o_ready);
        umma::mma_commit(&B.empty[tq % kSlots]);
        // MMA4: St (+)= Kw^T V
        if (!mbar_wait_abortable(B.kw_ready, ph, s_abort, kWaitNs, __LINE__)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16(tmem + kColSt, umma::desc_mnmajor(k_addr, ks), umma::desc_mnmajor(v_addr, ks),
                         idesc_nn, (i > 0) || has_in || (ks > 0));
        umma::mma_commit(B.st_ready);
        umma::mma_commit(&B.empty[tk % kSlots]);
        umma::mma_commit(&B.empty[tv % kSlots]);
      }
    }
  } else {
    // ------------------------------------------------------------ compute group
    // 256 threads: thread = (row r, column half).  A warp may only touch the
    // TMEM lane quarter (warp % 4), so the two warps that share a quarter split
    // the 128 columns between them.
    const int q4 = warp & 3;                 // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;        // 0: columns 0..63, 1: columns 64..127
    const int r = q4 * 32 + lane;            // row of the chunk / lane of TMEM
    const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
    const float g_row = s_pow[r + 1];        // g^(r+1)
    const float g_col = s_pow[kC - 1 - r];   // g^(C-1-r)
    const float g_chunk = s_pow[kC];         // g^C
    unsigned char* o_tile = smem + kOffO;
    unsigned char* sb_tile = smem + kOffSb;
    uint32_t va[32], vb[32];
    uint32_t wg_phase = 0;
    // write 32 packed columns [col0, col0+32) of row r into a swizzled tile
    auto store_block = [&](unsigned char* tile, int col0, const uint32_t (&w)[16]) {
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8)
        *reinterpret_cast<uint4*>(tile + umma::tile_chunk_offset(r, col0 + c8 * 8)) =
            make_uint4(w[4 * c8], w[4 * c8 + 1], w[4 * c8 + 2], w[4 * c8 + 3]);
    };
    for (int i = 0; i < nchunk; ++i) {
      const uint32_t ph = i & 1;
      bool ok = mbar_wait_abortable(B.s_ready, ph, s_abort, kWaitNs, __LINE__);
      if (!__all_sync(0xffffffffu, ok)) break;
      umma::fence_after_sync();
      // (a) P = bf16(S . decay), packed into TMEM over S: one table load and one
      // multiply per element (the table is 0 for negative exponents = masked).
      {
        const int cb0 = half * 2, cb1 = cb0 + 1;
        if (cb0 <= q4) umma::tmem_ld32(lane_base + kColS + cb0 * 32, va);  // warp-uniform:
        if (cb1 <= q4) umma::tmem_ld32(lane_base + kColS + cb1 * 32, vb);  // blocks right of the
        if (cb0 <= q4) umma::tmem_wait_ld();                               // diagonal are zero
        auto decay_block = [&](int cb, const uint32_t (&v)[32]) {
          uint32_t w[16];
          if (cb <= q4) {
            const float* pw = s_pow + (r - cb * 32);  // exponent of the block's first column
#pragma unroll
            for (int j = 0; j < 32; j += 2)
              w[j >> 1] = pack_bf16x2(__uint_as_float(v[j]) * pw[-j], __uint_as_float(v[j + 1]) * pw[-j - 1]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = 0u;
          }
          umma::tmem_st16(lane_base + kColS + p_col(cb * 32), w);
        };
        decay_block(cb0, va);
        decay_block(cb1, vb);
        umma::tmem_wait_st();
      }
      // The staging tile of the previous chunk's output must have been read by
      // its TMA store before (c) rewrites it; making the issuing thread wait
      // here, before its p_ready arrival, orders that ahead of MMA2 and hence
      // ahead of every thread's o_ready wait.
      if (tid == 64) bulk_wait_read<0>();
      umma::fence_before_sync();
      mbar_arrive(B.p_ready);
      // (d) state pass of the previous chunk, placed here so that it runs while
      // MMA2 (P.V) of this chunk executes and MMA3 (Q.Sb) can follow it directly:
      // Sb_i = bf16(St);  St <- g^C St  (ready for this chunk's MMA4)
      if (i > 0 || has_in) {
        const int cb0 = half * 2;
        if (i > 0) {
          ok = mbar_wait_abortable(B.st_ready, (i - 1) & 1, s_abort, kWaitNs, __LINE__);
          if (!__all_sync(0xffffffffu, ok)) break;
          umma::fence_after_sync();
          umma::tmem_ld32(lane_base + kColSt + cb0 * 32, va);
          umma::tmem_ld32(lane_base + kColSt + cb0 * 32 + 32, vb);
          umma::tmem_wait_ld();
        } else {
          // first chunk of a later segment: the state comes from the predecessor CTA
          // (prestaged: every segment's start state was computed before this launch)
          if (!prestaged) {
            const int* flag = seg_flag + size_t(seg - 1) * n_bh + bh;
            ok = wait_flag_abortable(flag, s_abort, kWaitNs, __LINE__);
            if (!__all_sync(0xffffffffu, ok)) break;
          }
          load_start_state(seg_state, seg, n_bh, bh, r, cb0, prestaged ? pieces_per_seg : 0,
                           powf(g, float(piece_rows)), va, vb);
        }
        auto state_block = [&](int cb, uint32_t (&v)[32]) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2)
            w[j >> 1] = pack_bf16x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
          store_block(sb_tile, cb * 32, w);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * g_chunk);
          umma::tmem_st32(lane_base + kColSt + cb * 32, v);
        };
        state_block(cb0, va);
        state_block(cb0 + 1, vb);
        umma::tmem_wait_st();
        umma::fence_before_sync();
        fence_proxy_async_smem();
        mbar_arrive(B.sb_ready);
      }
      // (b) K_i <- K_i . g^(C-1-r), in place (MMA1 has finished reading it);
      // this thread owns the 8 chunks of row r that lie in its column half.
      {
        unsigned char* k_tile = smem + kOffRing + ((3 * i) % kSlots) * kTile;
        uint4 x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          x[j] = *reinterpret_cast<const uint4*>(k_tile + umma::tile_chunk_offset(r, half * 64 + j * 8));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          x[j].x = pack_bf16x2(bf16lo_to_f32(x[j].x) * g_col, bf16hi_to_f32(x[j].x) * g_col);
          x[j].y = pack_bf16x2(bf16lo_to_f32(x[j].y) * g_col, bf16hi_to_f32(x[j].y) * g_col);
          x[j].z = pack_bf16x2(bf16lo_to_f32(x[j].z) * g_col, bf16hi_to_f32(x[j].z) * g_col);
          x[j].w = pack_bf16x2(bf16lo_to_f32(x[j].w) * g_col, bf16hi_to_f32(x[j].w) * g_col);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(k_tile + umma::tile_chunk_offset(r, half * 64 + j * 8)) = x[j];
      }
      fence_proxy_async_smem();
      mbar_arrive(B.kw_ready);
      // (c) o_i = (O1 + g^(r+1) O2) / scale, staged in shared memory in the
      // swizzled layout the TMA store expects
      ok = mbar_wait_abortable(B.o_ready, ph, s_abort, kWaitNs, __LINE__);
      if (!__all_sync(0xffffffffu, ok)) break;
      umma::fence_after_sync();
#pragma unroll 1
      for (int cbi = 0; cbi < 2; ++cbi) {
        const int cb = half * 2 + cbi;
        umma::tmem_ld32(lane_base + kColO1 + cb * 32, va);
        if (i > 0 || has_in) umma::tmem_ld32(lane_base + kColO2 + cb * 32, vb);
        umma::tmem_wait_ld();
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float lo = __uint_as_float(va[j]), hi = __uint_as_float(va[j + 1]);
          if (i > 0 || has_in) {
            lo = fmaf(g_row, __uint_as_float(vb[j]), lo);
            hi = fmaf(g_row, __uint_as_float(vb[j + 1]), hi);
          }
          w[j >> 1] = pack_bf16x2(lo * inv_scale, hi * inv_scale);
        }
        store_block(o_tile, cb * 32, w);
      }
      umma::fence_before_sync();
      mbar_arrive(B.o_free);
      fence_proxy_async_smem();
      mbar_arrive(B.wg_sync);
      ok = mbar_wait_abortable(B.wg_sync, wg_phase, s_abort, kWaitNs, __LINE__);
      wg_phase ^= 1;
      if (!__all_sync(0xffffffffu, ok)) break;
      if (tid == 64) {  // whole tile written: two {64 x 128} boxes go out asynchronously
        const int row = (chunk0 + i) * kC;   // the store is clipped at T
        umma::tma_store_3d(&map_o, 0, row, bh, o_tile);
        if (dv > 64) umma::tma_store_3d(&map_o, 64, row, bh, o_tile + umma::kSubTileBytes);
        bulk_commit();
      }
    }
    // hand the state to the next segment of this head: St after the last MMA4
    if (seg + 1 < n_seg && !prestaged) {
      bool ok = mbar_wait_abortable(B.st_ready, (nchunk - 1) & 1, s_abort, kWaitNs, __LINE__);
      if (__all_sync(0xffffffffu, ok)) {
        umma::fence_after_sync();
        const int cb0 = half * 2;
        umma::tmem_ld32(lane_base + kColSt + cb0 * 32, va);
        umma::tmem_ld32(lane_base + kColSt + cb0 * 32 + 32, vb);
        umma::tmem_wait_ld();
        float4* dst = reinterpret_cast<float4*>(seg_state + (size_t(seg) * n_bh + bh) * (kC * kC) + r * kC + cb0 * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __stcg(dst + j, make_float4(__uint_as_float(va[4 * j]), __uint_as_float(va[4 * j + 1]),
                                      __uint_as_float(va[4 * j + 2]), __uint_as_float(va[4 * j + 3])));
          __stcg(dst + 8 + j, make_float4(__uint_as_float(vb[4 * j]), __uint_as_float(vb[4 * j + 1]),
                                          __uint_as_float(vb[4 * j + 2]), __uint_as_float(vb[4 * j + 3])));
        }
        __threadfence();
        mbar_arrive(B.wg_sync);
        ok = mbar_wait_abortable(B.wg_sync, wg_phase, s_abort, kWaitNs, __LINE__);
        wg_phase ^= 1;
        if (ok && tid == 64) {
          int* flag = seg_flag + size_t(seg) * n_bh + bh;
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
        }
      }
    }
    if (tid == 64) bulk_wait_all<0>();  // the staged output has left shared memory
  }

  // Teardown: everyone meets, the last MMA4 is drained, TMEM goes back.
  __syncwarp();
  if (warp == 1 && lane == 0 && !*s_abort && nchunk > 0) {
    // the final commit (st_ready of the last chunk) covers every MMA issued
    mbar_wait_abortable(B.st_ready, (nchunk - 1) & 1, s_abort, kWaitNs, __LINE__);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  if (tid == 0 && *s_abort && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT | (*s_abort << 8));   // which wait: its source line
  if (warp == 1) {
    __syncwarp();
    umma::tmem_dealloc(tmem, 512);
  }
}

}  // namespace

bool decayed_tc_supported(int B, int H, int T, int dk, int dv, int C, int dtype) {
  // TMA row coordinates are 32-bit signed
  (void)C;  // the result is independent of the chunk size: 128-row chunks are used
  return dtype == CB2_BF16 && dk >= 8 && dk <= kC && dk % 8 == 0 && dv >= 8 && dv <= kC && dv % 8 == 0 &&
         T >= 1 && T < (1 << 30) && int64_t(B) * H < (int64_t(1) << 31);
}

// Segments per head: the smallest count in {1, 2, 4, 8} that fills the last wave
// of CTAs to 97 % (or the best of them), keeping at least 4 chunks per segment.
int decayed_tc_segments(int n_bh, int nchunk, int sms) {
  // a head's segments run one after the other, so cutting only pays when there is
  // more than one wave of heads to balance
  if (n_bh <= sms) return 1;
  int best = 1;
  double best_eff = 0.0;
  for (int n = 1; n <= 8; n *= 2) {
    if (nchunk % n != 0 || nchunk / n < 4) break;
    const double waves = double(n_bh) * n / sms;
    const double eff = waves / double((long long)((waves + 0.999999)));
    if (eff > best_eff + 1e-9) { best_eff = eff; best = n; }
    if (eff >= 0.97) break;
  }
  return best;
}

int decayed_seg_states_run(const void* k, const void* v, const float* gamma, int B, int H, int T, int dk,
                           int dv, int n_seg, int sub, float* seg_state, int* dev_status, cudaStream_t st);

// Parallel segments per head when heads are fewer than half the SMs: the largest power of
// two that keeps all CTAs in one wave, divides the chunk count and leaves four chunks or
// more per segment; 1 = not worth it (below 16 chunks the two extra launches cost more
// than the idle SMs: 8 chunks measured 29 us in one pass, 41 us cut in four).  The segments' start states are computed first
// (decayed_seg_state.cu), so the segments do not wait for one another.
int decayed_tc_parallel_segments(int n_bh, int nchunk, int sms) {
  if (n_bh * 2 > sms || nchunk < 16) return 1;
  int best = 1;
  for (int n = 2; n <= 16; n *= 2) {
    if (n_bh * n > sms || nchunk % n != 0 || nchunk / n < 4) break;
    best = n;
  }
  return best;
}

// How the start states of n parallel segments are prepared.  With at most four pieces to fold,
// the pre-pass writes the end state of every piece and each attention CTA folds the pieces before
// its segment itself (no scan launch); the pieces are then made as short as one wave of CTAs
// allows (`sub` per segment), because the pre-pass is a chain of chunk latencies too.  With more
// pieces a scan kernel turns end states into start states (sub = 0).
int decayed_tc_pieces_per_segment(int n_bh, int nchunk, int n_seg, int sms) {
  if (n_seg <= 1 || n_seg - 1 > 4) return 0;    // (folding 7 pieces in every CTA measured slower than the scan launch: 81 vs 63 us at 16 heads)
  const int per = nchunk / n_seg;
  int sub = 1;
  while ((n_seg - 1) * sub * 2 <= 4 && n_bh * (n_seg - 1) * sub * 2 <= sms && per % (sub * 2) == 0 &&
         per / (sub * 2) >= 4)
    sub *= 2;
  return sub;
}

// A quarter to half as many heads as SMs, long sequences: two CTAs per head in ONE launch with no
// scratch — the second walks the first's chunks for their state only (K and V: about half the time
// of a full chunk when the GPU is busy) before producing the rest, so the split sits past the
// middle; split points are even, so that the two Q slots of the ring keep alternating.
// Bit-identical to one CTA per head.  ways == 0: not this case.
SelfSplit decayed_tc_self_split(int n_bh, int nchunk, int sms) {
  SelfSplit sp{0, {0, 0, 0, 0, 0}};
  if (n_bh * 2 > sms || nchunk < 16) return sp;
  if (n_bh * 4 > sms) {
    // measured at 64 heads x 64 chunks: split 28: 143 us, 36: 135, 40: 131, 44: 125, 48: 131, 56: 150
    const int split = 2 * ((nchunk * 11 + 16) / 32);     // about 0.69 of the chunks
    if (split < 2 || split > nchunk - 2) return sp;
    sp.ways = 2;
    sp.s[1] = split;
    sp.s[2] = nchunk;
    return sp;
  }
  // (four CTAs per head for an eighth to a quarter as many heads as SMs, split at 0.57 / 0.83 / 0.95 of
  // the chunks, measured 102 us at 32 heads x 64 chunks against 93 us for parallel segments from a
  // pre-pass: the state-only walks re-read too much)
  return sp;
}

namespace {
int device_sms() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}
}  // namespace

// Scratch that lets heads be cut into segments: (n_seg - 1) * B*H states of
// 128 x 128 fp32, then as many flags.
size_t decayed_tc_scratch_bytes(int B, int H, int T) {
  const int nchunk = (T + kC - 1) / kC;
  if (decayed_tc_self_split(B * H, nchunk, device_sms()).ways > 0) return 0;
  const int n_par = decayed_tc_parallel_segments(B * H, nchunk, device_sms());
  if (n_par > 1) {
    const int sub = decayed_tc_pieces_per_segment(B * H, nchunk, n_par, device_sms());
    return size_t(n_par - 1) * (sub > 0 ? sub : 1) * B * H * (size_t(kC) * kC * sizeof(float) + sizeof(int));
  }
  const int n_seg = decayed_tc_segments(B * H, (T + kC - 1) / kC, device_sms());
  return size_t(n_seg - 1) * B * H * (size_t(kC) * kC * sizeof(float) + sizeof(int));
}

// How a call of these sizes is cut into CTAs (with the scratch decayed_tc_scratch_bytes asks for):
// 0 one CTA per head; 1 segments of a head handing their state over in scratch (more heads than SMs);
// 2 parallel segments from start states computed by a pre-pass; 3 two CTAs per head, the second
// accumulating the first's state by itself (no scratch).
int decayed_tc_plan(int B, int H, int T) {
  const int nchunk = (T + kC - 1) / kC, n_bh = B * H, sms = device_sms();
  if (decayed_tc_self_split(n_bh, nchunk, sms).ways > 0) return 3;
  if (decayed_tc_parallel_segments(n_bh, nchunk, sms) > 1) return 2;
  return decayed_tc_segments(n_bh, nchunk, sms) > 1 ? 1 : 0;
}

int decayed_tc_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B,
                   int H, int T, int dk, int dv, int C, float scale, void* scratch, size_t scratch_bytes,
                   int* dev_status, cudaStream_t st) {
  (void)C;
  // one map row = one position of one head; the head axis is the third coordinate, so
  // a ragged last chunk is zero-filled on load and clipped on store per head
  const uint64_t heads = uint64_t(B) * H;
  CUtensorMap mq, mk, mv, mo;
  int rc = umma::make_map_3d(&mq, q, true, dk, T, heads, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mk, k, true, dk, T, heads, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mv, v, true, dv, T, heads, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mo, o, true, dv, T, heads, 64, 128, true);
  if (rc != CB2_OK) return rc;
  // per device, so set on every call (cheap) rather than cached per process
  if (cudaFuncSetAttribute(decayed_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           int(kSmemBytes)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  const int n_bh = B * H;
  const int nchunk = (T + kC - 1) / kC;
  // several CTAs per head, each accumulating the state of the chunks before its own by itself: one
  // launch, no scratch
  const SelfSplit none{0, {0, 0, 0, 0, 0}};
  const SelfSplit self = decayed_tc_self_split(n_bh, nchunk, device_sms());
  if (self.ways > 0) {
    decayed_tc_kernel<<<n_bh * self.ways, kThreads, kSmemBytes, st>>>(mq, mk, mv, mo, gamma, H, T, dv, 1.0f / scale,
                                                                     n_bh, 1, nullptr, nullptr, 1, 0, 0, self,
                                                                     dev_status);
    CB2_LAUNCH_CHECK();
    return CB2_OK;
  }
  // few heads: parallel segments, start states computed up front
  const int n_par = decayed_tc_parallel_segments(n_bh, nchunk, device_sms());
  const int sub = decayed_tc_pieces_per_segment(n_bh, nchunk, n_par, device_sms());
  if (n_par > 1 && scratch && aligned16(scratch) &&
      scratch_bytes >= size_t(n_par - 1) * (sub > 0 ? sub : 1) * n_bh * size_t(kC) * kC * sizeof(float)) {
    float* states = static_cast<float*>(scratch);
    rc = decayed_seg_states_run(k, v, gamma, B, H, T, dk, dv, n_par, sub, states, dev_status, st);
    if (rc != CB2_OK) return rc;
    const int piece_rows = sub > 0 ? nchunk / n_par / sub * kC : 0;
    decayed_tc_kernel<<<n_bh * n_par, kThreads, kSmemBytes, st>>>(mq, mk, mv, mo, gamma, H, T, dv, 1.0f / scale,
                                                                 n_bh, n_par, states, nullptr, 1, sub, piece_rows,
                                                                 none, dev_status);
    CB2_LAUNCH_CHECK();
    return CB2_OK;
  }
  int n_seg = decayed_tc_segments(n_bh, (T + kC - 1) / kC, device_sms());
  const size_t state_bytes = size_t(n_seg - 1) * n_bh * size_t(kC) * kC * sizeof(float);
  const size_t flag_bytes = size_t(n_seg - 1) * n_bh * sizeof(int);
  if (n_seg > 1 && (!scratch || !aligned16(scratch) || scratch_bytes < state_bytes + flag_bytes ||
                    int64_t(n_bh) * n_seg >= (int64_t(1) << 31)))
    n_seg = 1;   // no room for the hand-off: one CTA per head
  float* seg_state = static_cast<float*>(scratch);
  int* seg_flag = n_seg > 1 ? reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + state_bytes) : nullptr;
  if (n_seg > 1 && cudaMemsetAsync(seg_flag, 0, flag_bytes, st) != cudaSuccess) return CB2_LAUNCH_FAIL;
  decayed_tc_kernel<<<n_bh * n_seg, kThreads, kSmemBytes, st>>>(mq, mk, mv, mo, gamma, H, T, dv, 1.0f / scale,
                                                               n_bh, n_seg, seg_state, seg_flag, 0, 0, 0,
                                                               none, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
