// Chunked decayed attention for fp32 tensors on the tensor cores (dk, dv <= 64):
//
//   o[t] = sum_{s<=t} g^(t-s) (q_t . k_s) v_s / scale          per (batch, head)
//
// (ChunkedDecayModule, catopt_carriers/decayed_lower.py:671-700) evaluated with
// the state-carry recurrence over 128-row chunks, a persistent CTA per SM taking
// (batch, head) units one after the other:
//   S    = Q K^T                                   (MMA1, 128 x 128 x dk)
//   O2   = Q St          St = state before the chunk, [dk x dv]   (MMA4)
//   P    = tril(S . g^(r-c))                       (score warps, in registers)
//   O1   = P V                                     (MMA2, 128 x dv x 128)
//   D    = V^T (K . g^(127-c))                     (MMA3, dv x dk x 128) = transposed state increment
//   o    = (O1 + g^(r+1) O2) / scale ,  St <- g^128 St + D^T
// A single TF32 pass keeps 10 mantissa bits, far from the 1e-5 this path
// promises, so every product is taken in three passes on operands split into
//   hi = the fp32 value itself (the tensor core reads its upper 19 bits, i.e. truncates it to TF32),
//   lo = value - truncated value (exact in fp32):
//   hi.hi + hi.lo + lo.hi, accumulated in fp32 tensor memory.
// The state itself is carried in fp32 by warps 2-5 (its hi tile is the fp32
// state), so its error does not grow with the number of chunks.
//
// Shared memory (224 KiB, one CTA per SM), 32 KiB tiles of 128 rows x 64 fp32 as
// two 128-byte-swizzled sub-tiles of 32 columns (what a TMA box {32, 128}
// writes): K of even chunks | K lo | K of odd chunks | V | V lo | Q (later the
// staged output), and the state hi | lo tiles (64 x 64).  K is loaded a whole
// chunk ahead into the tile the chunk before last has left, so that only the lo
// tile has to be built between two chunks.
// A tf32 operand whose rows run along the reduction (V in MMA2, V and K in MMA3:
// "MN-major") must sit in the 128-byte swizzle with 32-byte atoms: V's tensor
// map asks the TMA for that pattern, and the K rescale moves each row's chunks
// from the 16-byte-atom pattern MMA1 needs to that one (a permutation inside the
// row's 128 bytes, so each thread stays within the row it owns).
// Tensor memory (512 columns): S / P hi 0-127, P lo 128-255, O1 256-319,
// O2 320-383, Q hi 384-447 (reused for D once MMA4 has run), Q lo 448-511.  Q and
// P are A operands taken from tensor memory: an MMA with both tf32 operands in
// shared memory would need more than the 128 B/clk its port delivers.
// Measured cost of one tcgen05.mma kind::tf32 with an 8-deep step: 66 cycles at
// N = 128, 46 at N = 64 (M = 64 and M = 128 alike): 7.1 k cycles of tensor pipe
// per chunk at dk = dv = 64.
//
// Roles: warp 0 loads tiles with TMA; warp 1 issues the MMAs (MMA1 — its two
// products against K itself as soon as K has landed, the one against K lo when
// that tile is built —, MMA4, MMA3, MMA2: the state increment keeps the pipe busy
// while P is being built); warps 2-5 put Q into tensor memory, build half of K lo,
// carry the state and, once MMA1 has read K, rescale K for the state increment;
// warps 6-9 build the other half of K lo, write the output of the chunk before,
// build V lo, and mask and decay S into P.
// Every wait is bounded: on expiry the CTA records CB2_WAIT_TIMEOUT and leaves.
#include <algorithm>

#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kC = 128;
constexpr int kThreads = 320;
constexpr uint32_t kSub = 128 * 128;           // 128 rows x 32 fp32
constexpr uint32_t kTile = 2 * kSub;           // 128 rows x 64 fp32
constexpr uint32_t kSubS = 64 * 128;           // state sub-tile: 64 rows x 32 fp32
constexpr uint32_t kOffK0 = 0;                 // K of even chunks | K lo | K of odd chunks: a chunk's K and
constexpr uint32_t kOffKlo = kTile;            // the lo tile are neighbours either way
constexpr uint32_t kOffK1 = 2 * kTile;
constexpr uint32_t kOffVhi = 3 * kTile;
constexpr uint32_t kOffVlo = 4 * kTile;
constexpr uint32_t kOffQ = 5 * kTile;          // Q, then the staged output
constexpr uint32_t kOffShi = 6 * kTile;
constexpr uint32_t kOffSlo = kOffShi + 2 * kSubS;
constexpr uint32_t kOffBars = 7 * kTile;       // 224 KiB of tiles
constexpr int kNumBars = 16;
constexpr uint32_t kOffPow = kOffBars + kNumBars * 8;      // g^0 .. g^31 of the current unit
constexpr uint32_t kOffMisc = kOffPow + 132 * 4;
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;
static_assert(kSmemBytes <= 232448, "shared memory of one CTA");

constexpr uint32_t kColS = 0, kColPlo = 128, kColO1 = 256, kColO2 = 320, kColQhi = 384, kColQlo = 448;
constexpr uint32_t kColD = kColQhi;

struct Bars {
  uint64_t *q_full, *k_full, *v_full;      // TMA -> operand warps (k_full[2]: one per K tile)
  uint64_t *q_ready, *k_ready, *v_ready;   // operand warps -> MMA
  uint64_t* k2_ready;                      // K rescaled for the state increment
  uint64_t* s_ready;                       // MMA1 done
  uint64_t* p_ready;                       // P in tensor memory
  uint64_t* c_done;                        // every MMA of the chunk done (frees K lo, V and this chunk's K tile)
  uint64_t* st_ready;                      // state tiles written
  uint64_t* o_free;                        // O1 / O2 read
  uint64_t* wg_sync;                       // among the score warps
  uint64_t* spare;
  uint64_t* qtile_free;                    // the staged output has left the Q tile
};

__host__ __device__ constexpr uint32_t instr_desc_tf32(uint32_t M, uint32_t N, bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16) |
         ((N >> 3) << 17) | ((M >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
// A operand from tensor memory: lane = row, one tf32 per column, 8 columns per 8-deep step.
__device__ __forceinline__ void mma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}

// What a tf32 operand loses: v minus v truncated to TF32 (exact in fp32).
__device__ __forceinline__ float tf32_rest(float v) {
  return v - __uint_as_float(__float_as_uint(v) & 0xffffe000u);
}
__device__ __forceinline__ float4 rest4(const float4 v) {
  return make_float4(tf32_rest(v.x), tf32_rest(v.y), tf32_rest(v.z), tf32_rest(v.w));
}
// Byte offset of 16-byte chunk j (0..15) of `row` in a two-sub-tile swizzled tile.
__device__ __forceinline__ uint32_t chunk_off(uint32_t row, uint32_t j, uint32_t sub_bytes) {
  return (j >> 3) * sub_bytes + row * 128u + (((j & 7u) ^ (row & 7u)) << 4);
}
// Same for the 128-byte swizzle with 32-byte atoms: 32-byte chunk c of a row sits at c ^ (row % 4).
__device__ __forceinline__ uint32_t chunk_off32(uint32_t row, uint32_t j, uint32_t sub_bytes) {
  return (j >> 3) * sub_bytes + row * 128u + ((((((j & 7u) >> 1) ^ (row & 3u)) << 1) | (j & 1u)) << 4);
}
// Rows r and r + 4 of that pattern keep a given chunk in the same banks, so a quarter-warp writing
// chunk j of eight consecutive rows would hit every bank twice: lanes 4-7 of each eight take the
// two chunks of a 32-byte pair in the other order.  x holds the eight chunks of columns
// [32 half, 32 half + 32) of `row`; REST also writes their truncation remainders to the lo tile.
template <bool REST>
__device__ __forceinline__ void store_half_32b(unsigned char* hi_tile, unsigned char* lo_tile, uint32_t row,
                                               int half, const float4 (&x)[8], uint32_t sub_bytes) {
  const bool flip = (row >> 2) & 1u;
#pragma unroll
  for (int pr = 0; pr < 4; ++pr) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      // t-th store of the pair: chunk 2 pr + (t ^ flip)
      const float4 a = x[2 * pr + t], b = x[2 * pr + (t ^ 1)];
      const float4 v = flip ? b : a;
      const uint32_t off = chunk_off32(row, half * 8 + 2 * pr + (t ^ int(flip)), sub_bytes);
      *reinterpret_cast<float4*>(hi_tile + off) = v;
      if (REST) *reinterpret_cast<float4*>(lo_tile + off) = rest4(v);
    }
  }
}
// Shared-memory matrix descriptor with the layout type given (2: 128-byte swizzle, 1: 128-byte swizzle
// with 32-byte atoms).
__device__ __forceinline__ uint64_t smem_desc_lt(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                 uint32_t layout_type) {
  return uint64_t((smem_addr & 0x3ffffu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) |
         (uint64_t(sbo_bytes >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(layout_type) << 61);
}
// K-major operand, 8-deep step ks of a swizzled tile: 8-row groups 1024 B apart, the step advances
// 32 B inside the 128-byte row and moves to the second sub-tile after four steps.
__device__ __forceinline__ uint64_t desc_k(uint32_t tile_addr, int ks, uint32_t sub_bytes) {
  return umma::smem_desc(tile_addr + (ks >> 2) * sub_bytes + (ks & 3) * 32u, 16u, 1024u);
}
// MN-major operand (32-byte-atom swizzle), 8-deep step ks: the 8 K-rows of the step are two groups of
// four rows, 512 B apart (stride offset); the second 32 MN elements sit in the second sub-tile
// (leading offset).
__device__ __forceinline__ uint64_t desc_mn(uint32_t tile_addr, int ks) {
  return smem_desc_lt(tile_addr + ks * 1024u, kSub, 512u, 1u);
}

__global__ void __launch_bounds__(kThreads, 1)
decayed_tf32_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                    const float* __restrict__ gamma, int H, int T, int dk, int dv, float inv_scale, int n_bh,
                    int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  float* s_diag = reinterpret_cast<float*>(smem + kOffPow);    // g^0 .. g^31 of the head being scored
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 4);
  const Bars B{bars,     bars + 1, bars + 3,  bars + 4,  bars + 5,  bars + 6,  bars + 7,
               bars + 8, bars + 9, bars + 10, bars + 11, bars + 12, bars + 13, bars + 14, bars + 15};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nchunk = (T + kC - 1) / kC;
  const int nks = (dk + 7) / 8;                 // 8-deep steps over the key dimension
  // Persistent CTA: units blockIdx.x, blockIdx.x + gridDim.x, ... one after the other as ONE stream of
  // chunks (index t), so that the loads, the output of the last chunk and the first products of the
  // next unit overlap; only the state restarts at a unit's first chunk.
  const int n_mine = (n_bh - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
  const int total = n_mine * nchunk;

  if (tid == 0) {
    mbar_init(B.q_full, 1);
    mbar_init(&B.k_full[0], 1);
    mbar_init(&B.k_full[1], 1);
    mbar_init(B.v_full, 1);
    mbar_init(B.q_ready, 128);
    mbar_init(B.k_ready, 256);
    mbar_init(B.v_ready, 128);
    mbar_init(B.k2_ready, 128);
    mbar_init(B.s_ready, 1);
    mbar_init(B.p_ready, 128);
    mbar_init(B.c_done, 1);
    mbar_init(B.st_ready, 128);
    mbar_init(B.o_free, 128);
    mbar_init(B.wg_sync, 128);
    mbar_init(B.spare, 1);
    mbar_init(B.qtile_free, 1);
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    __syncwarp();
    umma::tmem_alloc(s_tmem, 512);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *s_tmem;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      umma::tma_prefetch_desc(&map_q);
      umma::tma_prefetch_desc(&map_k);
      umma::tma_prefetch_desc(&map_v);
      umma::tma_prefetch_desc(&map_o);
      int nq = 0, nv = 0, nk0 = 0, nk1 = 0;       // copies issued per barrier
      // rows past T arrive as zeros
      // each of the three load streams keeps its own (chunk, unit) position: no division per load
      struct Pos { int ci, bh; };
      const int step = int(gridDim.x);
      auto advance = [&](Pos& p) {
        if (++p.ci == nchunk) { p.ci = 0; p.bh += step; }
      };
      Pos pq{0, int(blockIdx.x)}, pk{0, int(blockIdx.x)}, pv{0, int(blockIdx.x)};
      auto load_q = [&](int) {
        const int row = pq.ci * kC, bh = pq.bh;
        advance(pq);
        mbar_arrive_expect_tx(B.q_full, kTile);
        umma::tma_load_3d(smem + kOffQ, &map_q, 0, row, bh, B.q_full);
        umma::tma_load_3d(smem + kOffQ + kSub, &map_q, 32, row, bh, B.q_full);
        ++nq;
      };
      auto load_k = [&](int t) {
        const int row = pk.ci * kC, bh = pk.bh;
        advance(pk);
        const int b = t & 1;
        unsigned char* dst = smem + (b ? kOffK1 : kOffK0);
        mbar_arrive_expect_tx(&B.k_full[b], kTile);
        umma::tma_load_3d(dst, &map_k, 0, row, bh, &B.k_full[b]);
        umma::tma_load_3d(dst + kSub, &map_k, 32, row, bh, &B.k_full[b]);
        if (b) ++nk1; else ++nk0;
      };
      auto load_v = [&](int) {
        const int row = pv.ci * kC, bh = pv.bh;
        advance(pv);
        mbar_arrive_expect_tx(B.v_full, kTile);
        umma::tma_load_3d(smem + kOffVhi, &map_v, 0, row, bh, B.v_full);
        umma::tma_load_3d(smem + kOffVhi + kSub, &map_v, 32, row, bh, B.v_full);
        ++nv;
      };
      if (total > 0) {
        load_q(0);
        load_k(0);
        load_v(0);
      }
      if (total > 1) load_k(1);
      for (int t = 0; t + 1 < total; ++t) {
        // the Q tile is free once Q_t sits in tensor memory (first chunk) or the output of
        // chunk t-1, staged there, has left
        if (!(t == 0 ? mbar_wait_abortable(B.q_ready, 0, s_abort)
                     : mbar_wait_abortable(B.qtile_free, (t - 1) & 1, s_abort)))
          break;
        load_q(t + 1);
        // chunk t done: V and this chunk's K tile are free
        if (!mbar_wait_abortable(B.c_done, t & 1, s_abort)) break;
        load_v(t + 1);
        if (t + 2 < total) load_k(t + 2);
      }
      if (*s_abort) {
        // leaving early: let the copies in flight land first (bounded)
        if (nq) mbar_wait_bounded(B.q_full, (nq - 1) & 1);
        if (nv) mbar_wait_bounded(B.v_full, (nv - 1) & 1);
        if (nk0) mbar_wait_bounded(&B.k_full[0], (nk0 - 1) & 1);
        if (nk1) mbar_wait_bounded(&B.k_full[1], (nk1 - 1) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc_tf32(128, 128, false, false);
      constexpr uint32_t idesc_o2 = instr_desc_tf32(128, 64, false, false);
      constexpr uint32_t idesc_o1 = instr_desc_tf32(128, 64, false, true);
      constexpr uint32_t idesc_d = instr_desc_tf32(64, 64, true, true);
      constexpr uint32_t idesc_d2 = instr_desc_tf32(64, 128, true, true);
      // descriptors of step 0; a step adds a constant to the start-address field (a lone thread issues
      // every MMA, so the issue loops are unrolled down to one add per MMA)
      const uint32_t k0 = smem_u32(smem + kOffK0);
      const uint64_t klo_k = desc_k(smem_u32(smem + kOffKlo), 0, kSub), klo_m = desc_mn(smem_u32(smem + kOffKlo), 0);
      const uint64_t shi_k = desc_k(smem_u32(smem + kOffShi), 0, kSubS), slo_k = desc_k(smem_u32(smem + kOffSlo), 0, kSubS);
      const uint64_t vhi_m = desc_mn(smem_u32(smem + kOffVhi), 0), vlo_m = desc_mn(smem_u32(smem + kOffVlo), 0);
      int ci = 0;                                // chunk within the unit
      uint32_t k2_phase = 0;                     // k2_ready skips a unit's last chunk, so it keeps its own count
      for (int t = 0; t < total; ++t, ci = (ci + 1 == nchunk ? 0 : ci + 1)) {
        const uint32_t ph = t & 1;
        const uint64_t khi_k = desc_k(k0 + ph * 2 * kTile, 0, kSub), khi_m = desc_mn(k0 + ph * 2 * kTile, 0);
        // K' hi and lo side by side as one 128-wide operand: hi | lo for even chunks, lo | hi for odd ones
        const uint64_t kboth_m = ph ? klo_m : khi_m;
        // MMA1: S = Q K^T.  The two products against K itself start as soon as Q is in tensor memory
        // and the K tile has landed; the one against K lo follows when the warps have built that tile.
        if (!mbar_wait_abortable(B.q_ready, ph, s_abort)) break;
        if (!mbar_wait_abortable(&B.k_full[ph], (t >> 1) & 1, s_abort)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          if (ks < nks) {
            const uint32_t off = ((ks >> 2) * kSub + (ks & 3) * 32u) >> 4;
            mma_tf32_ts(tmem + kColS, tmem + kColQlo + ks * 8, khi_k + off, idesc_s, ks > 0);
            mma_tf32_ts(tmem + kColS, tmem + kColQhi + ks * 8, khi_k + off, idesc_s, true);
          }
        }
        if (!mbar_wait_abortable(B.k_ready, ph, s_abort)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          if (ks < nks) {
            const uint32_t off = ((ks >> 2) * kSub + (ks & 3) * 32u) >> 4;
            mma_tf32_ts(tmem + kColS, tmem + kColQhi + ks * 8, klo_k + off, idesc_s, true);
          }
        }
        umma::mma_commit(B.s_ready);
        // MMA4: O2 = Q St
        if (!mbar_wait_abortable(B.st_ready, ph, s_abort)) break;
        if (t > 0 && !mbar_wait_abortable(B.o_free, (t - 1) & 1, s_abort)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          if (ks < nks) {
            const uint32_t off = ((ks >> 2) * kSubS + (ks & 3) * 32u) >> 4;
            mma_tf32_ts(tmem + kColO2, tmem + kColQlo + ks * 8, shi_k + off, idesc_o2, ks > 0);
            mma_tf32_ts(tmem + kColO2, tmem + kColQhi + ks * 8, slo_k + off, idesc_o2, true);
            mma_tf32_ts(tmem + kColO2, tmem + kColQhi + ks * 8, shi_k + off, idesc_o2, true);
          }
        }
        // MMA3: D = V^T K' (not needed after a unit's last chunk); lands where Q was.  Issued before
        // MMA2 so that the tensor pipe has work while the score warps build P.
        if (ci + 1 < nchunk) {
          if (!mbar_wait_abortable(B.v_ready, ph, s_abort)) break;
          if (!mbar_wait_abortable(B.k2_ready, k2_phase, s_abort)) break;
          k2_phase ^= 1;
          umma::fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 16; ++ks) {
            const uint32_t off = (ks * 1024u) >> 4;
            // V hi against [K' hi | K' lo] in one 128-wide MMA (two of the three products; the state warps
            // add the halves), then V lo against K' hi
            mma_tf32_ss(tmem + kColD, vhi_m + off, kboth_m + off, idesc_d2, ks > 0);
            mma_tf32_ss(tmem + kColD, vlo_m + off, khi_m + off, idesc_d, true);
          }
        }
        // MMA2: O1 = P V
        if (!mbar_wait_abortable(B.p_ready, ph, s_abort)) break;
        if (!mbar_wait_abortable(B.v_ready, ph, s_abort)) break;
        umma::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 16; ++ks) {
          const uint32_t off = (ks * 1024u) >> 4;
          mma_tf32_ts(tmem + kColO1, tmem + kColPlo + ks * 8, vhi_m + off, idesc_o1, ks > 0);
          mma_tf32_ts(tmem + kColO1, tmem + kColS + ks * 8, vlo_m + off, idesc_o1, true);
          mma_tf32_ts(tmem + kColO1, tmem + kColS + ks * 8, vhi_m + off, idesc_o1, true);
        }
        umma::mma_commit(B.c_done);
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- operand / state warps
    // Per chunk: read the state increment of the chunk before, put Q into tensor memory, build half of
    // K lo (-> MMA1 can finish), carry the state (-> MMA4), rescale K once MMA1 is done (-> MMA3).
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;                // row of every tile this thread owns
    const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
    unsigned char* qt = smem + kOffQ;
    unsigned char* kl = smem + kOffKlo;
    unsigned char* sh = smem + kOffShi;
    unsigned char* sl = smem + kOffSlo;
    float w = 0.f, gC = 0.f;                     // g^(127-r): decay of key r to the end of the chunk; g^128
    bool ok = true;
    int ci = 0, bh = int(blockIdx.x);
    for (int t = 0; ok && t < total; ++t, ++ci) {
      if (ci == nchunk) { ci = 0; bh += int(gridDim.x); }
      const uint32_t ph = t & 1;
      unsigned char* kh = smem + (ph ? kOffK1 : kOffK0);
      if (ci == 0) {
        const float g = gamma[bh % H];
        w = powf(g, float(kC - 1 - r));
        gC = powf(g, float(kC));
      }
      // every MMA of the chunk before is done: K lo and the Q columns are free
      if (t > 0) {
        ok = mbar_wait_abortable(B.c_done, (t - 1) & 1, s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        umma::fence_after_sync();
      }
      // D of the chunk before: two 64-column halves (products with K' hi and K' lo) to be added.  A
      // 64-row accumulator keeps row n in lane (n % 16) of lane quarter n / 16.  Read first: Q goes
      // into the same columns.
      float d[64];
      if (ci > 0) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t a[32], b[32];
          umma::tmem_ld32(lane_base + kColD + half * 32, a);
          umma::tmem_ld32(lane_base + kColD + 64 + half * 32, b);
          umma::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) d[half * 32 + j] = __uint_as_float(a[j]) + __uint_as_float(b[j]);
        }
      }
      // Q -> tensor memory (value, remainder)
      ok = mbar_wait_abortable(B.q_full, ph, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 v = *reinterpret_cast<const float4*>(qt + chunk_off(r, half * 8 + j, kSub));
          const float4 l = rest4(v);
          hi[4 * j] = __float_as_uint(v.x); hi[4 * j + 1] = __float_as_uint(v.y);
          hi[4 * j + 2] = __float_as_uint(v.z); hi[4 * j + 3] = __float_as_uint(v.w);
          lo[4 * j] = __float_as_uint(l.x); lo[4 * j + 1] = __float_as_uint(l.y);
          lo[4 * j + 2] = __float_as_uint(l.z); lo[4 * j + 3] = __float_as_uint(l.w);
        }
        umma::tmem_st32(lane_base + kColQhi + half * 32, hi);
        umma::tmem_st32(lane_base + kColQlo + half * 32, lo);
      }
      umma::tmem_wait_st();
      umma::fence_before_sync();
      mbar_arrive(B.q_ready);
      // K lo, columns 0-31 (the K tile itself is the hi operand; the other warpgroup does columns 32-63)
      ok = mbar_wait_abortable(&B.k_full[ph], (t >> 1) & 1, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      {
        // (all loads before the first store: the tiles may alias as far as the compiler knows, and a
        // load behind a store would wait for it)
        float4 x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = *reinterpret_cast<const float4*>(kh + chunk_off(r, j, kSub));
#pragma unroll
        for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(kl + chunk_off(r, j, kSub)) = rest4(x[j]);
      }
      fence_proxy_async_smem();
      mbar_arrive(B.k_ready);
      // state: St <- g^128 St + D^T (zero before a unit's first chunk); the hi tile is the fp32 state
      if (ci == 0) {
        for (int j = 0; j < 16; ++j)
          *reinterpret_cast<float4*>(sh + ((tid - 64) * 16 + j) * 16) = make_float4(0.f, 0.f, 0.f, 0.f);   // hi and lo
      } else if (lane < 16) {
        const uint32_t n = q4 * 16 + lane;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float4 a[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = *reinterpret_cast<const float4*>(sh + chunk_off(n, half * 8 + j, kSubS));
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int e = 4 * (half * 8 + j);
            const uint32_t off = chunk_off(n, half * 8 + j, kSubS);
            const float4 x = make_float4(fmaf(gC, a[j].x, d[e]), fmaf(gC, a[j].y, d[e + 1]),
                                         fmaf(gC, a[j].z, d[e + 2]), fmaf(gC, a[j].w, d[e + 3]));
            *reinterpret_cast<float4*>(sh + off) = x;
            *reinterpret_cast<float4*>(sl + off) = rest4(x);
          }
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(B.st_ready);
      // K' = K g^(127-r), moved to the 32-byte-atom pattern, once MMA1 has read K
      if (ci + 1 < nchunk) {
        ok = mbar_wait_abortable(B.s_ready, ph, s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float4 x[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 a = *reinterpret_cast<const float4*>(kh + chunk_off(r, half * 8 + j, kSub));
            x[j] = make_float4(a.x * w, a.y * w, a.z * w, a.w * w);
          }
          store_half_32b<true>(kh, kl, r, half, x, kSub);
        }
        fence_proxy_async_smem();
        mbar_arrive(B.k2_ready);
      }
    }
  } else {
    // ---------------------------------------------------------------- score / output warps
    // Per chunk: the other half of K lo, the output of the chunk before (-> MMA4 may overwrite O2), V lo
    // (-> MMA3), then P from S (-> MMA2).
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const int wt = tid - 192;                    // 0..127 among these warps
    const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
    unsigned char* kl = smem + kOffKlo;
    unsigned char* vh = smem + kOffVhi;
    unsigned char* vl = smem + kOffVlo;
    unsigned char* ot = smem + kOffQ;            // the output is staged where Q was
    float fcross = 0.f;                          // g^(r+1)
    float gp[32];                                // g^(31-j)
    float acb[3] = {0.f, 0.f, 0.f};              // g^(r - 32 cb - 31) for the key blocks before the diagonal one
    uint32_t wg_phase = 0;
    bool ok = true;
    auto wg_barrier = [&]() -> bool {
      mbar_arrive(B.wg_sync);
      bool fine = mbar_wait_abortable(B.wg_sync, wg_phase, s_abort);
      wg_phase ^= 1;
      return __all_sync(0xffffffffu, fine);
    };
    // o = (O1 + g^(r+1) O2) / scale of chunk `row / 128` of unit `bh`, staged as a swizzled tile where Q
    // was (the next Q is in tensor memory by then) and stored by TMA
    auto write_output = [&](int row, int bh, bool more) -> bool {
      if (wt == 0) bulk_wait_read<0>();          // the previous store has read the staging tile
      if (!wg_barrier()) return false;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t a[32], b[32];
        umma::tmem_ld32(lane_base + kColO1 + half * 32, a);
        umma::tmem_ld32(lane_base + kColO2 + half * 32, b);
        umma::tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o;
          o.x = (__uint_as_float(a[4 * j]) + fcross * __uint_as_float(b[4 * j])) * inv_scale;
          o.y = (__uint_as_float(a[4 * j + 1]) + fcross * __uint_as_float(b[4 * j + 1])) * inv_scale;
          o.z = (__uint_as_float(a[4 * j + 2]) + fcross * __uint_as_float(b[4 * j + 2])) * inv_scale;
          o.w = (__uint_as_float(a[4 * j + 3]) + fcross * __uint_as_float(b[4 * j + 3])) * inv_scale;
          *reinterpret_cast<float4*>(ot + chunk_off(r, half * 8 + j, kSub)) = o;
        }
      }
      umma::fence_before_sync();
      mbar_arrive(B.o_free);
      fence_proxy_async_smem();
      if (!wg_barrier()) return false;
      if (wt == 0) {
        umma::tma_store_3d(&map_o, 0, row, bh, ot);
        if (dv > 32) umma::tma_store_3d(&map_o, 32, row, bh, ot + kSub);
        bulk_commit();
        if (more) {
          bulk_wait_read<0>();
          mbar_arrive(B.qtile_free);             // the next but one Q may be loaded
        }
      }
      return true;
    };
    int ci = 0, bh = int(blockIdx.x), prev_row = 0, prev_bh = 0;
    for (int t = 0; ok && t < total; ++t, ++ci) {
      if (ci == nchunk) { ci = 0; bh += int(gridDim.x); }
      const uint32_t ph = t & 1;
      // K lo, columns 32-63 (every MMA of the chunk before is done: the loop ends on that wait)
      ok = mbar_wait_abortable(&B.k_full[ph], (t >> 1) & 1, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      {
        const unsigned char* kh = smem + (ph ? kOffK1 : kOffK0);
        float4 x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = *reinterpret_cast<const float4*>(kh + chunk_off(r, 8 + j, kSub));
#pragma unroll
        for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(kl + chunk_off(r, 8 + j, kSub)) = rest4(x[j]);
      }
      fence_proxy_async_smem();
      mbar_arrive(B.k_ready);
      // output of the chunk before, once this chunk's Q has left its tile
      if (t > 0) {
        ok = mbar_wait_abortable(B.q_ready, ph, s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        umma::fence_after_sync();
        if (!write_output(prev_row, prev_bh, true)) { ok = false; break; }
      }
      prev_row = ci * kC;
      prev_bh = bh;
      if (ci == 0) {
        // a new unit: its rate's powers (after the output above, which still belongs to the unit before)
        const float g = gamma[bh % H];
        if (wt < 32) s_diag[wt] = powf(g, float(wt));
        fcross = powf(g, float(r + 1));
#pragma unroll
        for (int cb = 0; cb < 3; ++cb) acb[cb] = cb < q4 ? powf(g, float(r - 32 * cb - 31)) : 0.f;
        if (!wg_barrier()) { ok = false; break; }
#pragma unroll
        for (int j = 0; j < 32; ++j) gp[j] = s_diag[31 - j];
      }
      // V lo (the TMA wrote V in the 32-byte-atom pattern already, and the tile itself is the hi operand)
      ok = mbar_wait_abortable(B.v_full, ph, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      {
        // (lanes 4-7 of each eight take the two chunks of a 32-byte pair in the other order: rows r and
        // r + 4 keep a chunk in the same banks)
        const uint32_t flip = (r >> 2) & 1u;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float4 x[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            x[j] = *reinterpret_cast<const float4*>(vh + chunk_off32(r, uint32_t(half * 8 + j) ^ flip, kSub));
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(vl + chunk_off32(r, uint32_t(half * 8 + j) ^ flip, kSub)) = rest4(x[j]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(B.v_ready);
      // P = tril(S . g^(r-c)) as value + remainder
      ok = mbar_wait_abortable(B.s_ready, ph, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      umma::fence_after_sync();
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t v[32], lo[32];
        if (cb > q4) {
          // every key of the block is after every row of this warp
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
          umma::tmem_st32(lane_base + kColS + cb * 32, v);
          umma::tmem_st32(lane_base + kColPlo + cb * 32, v);
          continue;
        }
        umma::tmem_ld32(lane_base + kColS + cb * 32, v);
        umma::tmem_wait_ld();
        if (cb < q4) {
          // all keys visible: g^(r-c) = g^(r - 32 cb - 31) g^(31-j)
          const float a = cb == 0 ? acb[0] : (cb == 1 ? acb[1] : acb[2]);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float p = __uint_as_float(v[j]) * (a * gp[j]);
            v[j] = __float_as_uint(p);
            lo[j] = __float_as_uint(tf32_rest(p));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int e = lane - j;             // r - c on the diagonal block
            const float p = e >= 0 ? __uint_as_float(v[j]) * s_diag[e] : 0.f;
            v[j] = __float_as_uint(p);
            lo[j] = __float_as_uint(tf32_rest(p));
          }
        }
        umma::tmem_st32(lane_base + kColS + cb * 32, v);
        umma::tmem_st32(lane_base + kColPlo + cb * 32, lo);
      }
      umma::tmem_wait_st();
      umma::fence_before_sync();
      mbar_arrive(B.p_ready);

      ok = mbar_wait_abortable(B.c_done, ph, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      umma::fence_after_sync();
    }
    if (ok && total > 0) write_output(prev_row, prev_bh, false);
    if (wt == 0) bulk_wait_all<0>();
  }
  __syncwarp();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  if (tid == 0 && *s_abort && dev_status) atomicExch(dev_status, CB2_WAIT_TIMEOUT);
  if (warp == 1) {
    __syncwarp();
    umma::tmem_dealloc(tmem, 512);
  }
}

// fp32 [heads, T, d] tensor, box {32, 128, 1}, 128-byte swizzle with 16-byte atoms (the usual one) or with
// 32-byte atoms (the pattern a tf32 operand whose rows run along the reduction must have).
int make_map(CUtensorMap* out, const void* base, uint64_t d, uint64_t T, uint64_t heads, bool atom32) {
  using Fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                          const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                          CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !p)
      return CB2_LAUNCH_FAIL;
    fn = reinterpret_cast<Fn>(p);
  }
  const cuuint64_t gdim[3] = {d, T, heads};
  const cuuint64_t gstride[2] = {d * 4, d * T * 4};
  const cuuint32_t box[3] = {32, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE,
            atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? CB2_OK
             : CB2_LAUNCH_FAIL;
}

int device_sms() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace

// fp32 tensors with both head dimensions at most 64 (multiples of 4, so that rows are 16-byte
// aligned for TMA) and enough (batch, head) units for one CTA each to be worth it: below about a
// sixth of the SMs the FMA path, which spreads a head's chunks over CTAs, is faster.
bool decayed_tf32_supported(int B, int H, int T, int dk, int dv, int dtype) {
  if (dtype != CB2_F32) return false;
  if (dk < 4 || dv < 4 || dk > 64 || dv > 64 || dk % 4 || dv % 4) return false;
  if (T < 1) return false;
  return int64_t(B) * H >= 24 && int64_t(B) * H < (int64_t(1) << 31);
}

int decayed_tf32_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B, int H,
                     int T, int dk, int dv, float scale, int* dev_status, cudaStream_t st) {
  const uint64_t heads = uint64_t(B) * H;
  CUtensorMap mq, mk, mv, mo;
  int rc = make_map(&mq, q, dk, T, heads, false);
  if (rc == CB2_OK) rc = make_map(&mk, k, dk, T, heads, false);
  if (rc == CB2_OK) rc = make_map(&mv, v, dv, T, heads, true);
  if (rc == CB2_OK) rc = make_map(&mo, o, dv, T, heads, false);
  if (rc != CB2_OK) return rc;
  if (cudaFuncSetAttribute(decayed_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           int(kSmemBytes)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  // one persistent CTA per SM walks its units one after the other
  const unsigned grid = unsigned(std::min<uint64_t>(heads, uint64_t(device_sms())));
  decayed_tf32_kernel<<<grid, kThreads, kSmemBytes, st>>>(mq, mk, mv, mo, gamma, H, T, dk, dv, 1.0f / scale,
                                                          int(heads), dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
