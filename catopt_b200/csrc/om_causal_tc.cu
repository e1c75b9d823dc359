// Softmax attention, causal or unmasked, on the tensor cores (bf16, dk, dv <= 128): the
// online-softmax monoid of the reference (`_om_elem` / `_om_compose`,
// catopt_torch/torch_bridge.py:1974-2006) folded over 128-key blocks, with the
// running (max, sum) pair in registers and the weighted sum in tensor memory.
//
// CTA = 128 queries of one (batch, head); two CTAs share an SM (each takes half
// of the tensor memory and of the shared memory), so one CTA's softmax runs
// while the other's products are on the tensor core.  Per key block j (causal:
// j <= i):
//   MMA1  S_j = Q K_j^T                         -> TMEM
//   WG    the row's 128 scores come to registers in one batch of TMEM loads;
//         m' = max(m, rowmax S_j); P = exp(S_j - m') as bf16, written over S_j;
//         l = l e^(m-m') + rowsum P;  O <- O e^(m-m').  The reference point m
//         follows the maximum lazily (only after it moved by 2^8), so the O
//         rescale is rare; a warp whose rows all kept theirs skips it
//   MMA2  O += P V_j      (A operand read from TMEM, V_j MN-major from its tile)
// and finally o = O / l through a staging tile and a TMA store.  Entirely masked
// blocks are never visited; a partially masked block (the diagonal one, or the
// last one when Tk is ragged) masks per element.  Thread = one query row (one
// TMEM lane), so the row maxima and sums need no cross-thread traffic.
//
// Roles: warp 0 = TMA producer (Q once, then K_j / V_j tiles alternating between
// two slots; 3-D tensor maps clip and zero-fill per head), warp 1 = MMA issuer
// and TMEM owner, warps 2..5 = softmax group.  Every wait is bounded.
#include "umma.cuh"

namespace cb2 {
namespace {

constexpr int kQ = 128;                   // queries per CTA = keys per block
constexpr int kSlots = 2;                 // slot 0: K_j, slot 1: V_j
constexpr int kThreads = 192;
constexpr uint32_t kTile = umma::kTileBytes;
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffRing = kTile;
constexpr uint32_t kOffO = kOffQ;         // the output is staged over Q once the last scores are out
constexpr uint32_t kOffBars = kOffRing + kSlots * kTile;
constexpr int kNumBars = 2 * kSlots + 5;
constexpr uint32_t kOffMisc = kOffBars + kNumBars * 8;
constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;   // 97.4 KiB: two CTAs per SM
constexpr uint32_t kColS = 0, kColO = 128;
constexpr uint32_t kTmemCols = 256;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// BIAS: with an additive attention bias (a separate instantiation, so that the plain kernel keeps
// its register budget)
template <bool BIAS>
__global__ void __launch_bounds__(kThreads, 2)
om_causal_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                    int Tq, int Tk, int dk, int dv, int n_bh, int causal, float scale_log2e, int key_offset,
                    const float* __restrict__ m_in, const float* __restrict__ l_in, const float* __restrict__ a_in,
                    float* __restrict__ m_out, float* __restrict__ l_out, float* __restrict__ a_out,
                    const OmBias bias, int* dev_status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  uint64_t* full = bars;                         // [kSlots] TMA -> MMA
  uint64_t* empty = bars + kSlots;               // [kSlots] MMA -> TMA
  uint64_t* q_full = bars + 2 * kSlots;
  uint64_t* s_ready = bars + 2 * kSlots + 1;     // MMA1 done
  uint64_t* p_ready = bars + 2 * kSlots + 2;     // P written, O rescaled (128 arrivals)
  uint64_t* o_done = bars + 2 * kSlots + 3;      // MMA2 done
  uint64_t* wg_sync = bars + 2 * kSlots + 4;     // barrier among the 128 softmax threads
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + kOffMisc + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTAs are handed out in launch order: the latest query blocks of EVERY head
  // first (they visit the most key blocks), the cheap early ones last, which keeps
  // the tail of the grid short
  const int bh = blockIdx.x % n_bh;
  const int qb = int(gridDim.x / n_bh) - 1 - int(blockIdx.x / n_bh);
  const int q0 = qb * kQ;
  // key blocks with at least one visible key (all of them without the causal mask): key j of
  // this call is hidden from query row t when key_offset + j > t.  Possibly none (a streaming
  // step whose keys all lie in the future of this query block).
  const int nkb_all = (Tk + kQ - 1) / kQ;
  const int last_vis = q0 + kQ - 1 - key_offset;           // last key the block's last row may see
  const int nkb = causal ? (last_vis < 0 ? 0 : min(nkb_all, last_vis / kQ + 1)) : nkb_all;
  const bool has_state = m_in != nullptr;                  // continue from the caller's carrier

  if (tid == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(q_full, 1);
    mbar_init(s_ready, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    mbar_init(wg_sync, 128);
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
  const uint32_t q_addr = smem_u32(smem + kOffQ);
  const uint32_t ring_addr = smem_u32(smem + kOffRing);

  if (warp == 0) {
    if (lane == 0) {
      umma::tma_prefetch_desc(&map_q);
      umma::tma_prefetch_desc(&map_k);
      umma::tma_prefetch_desc(&map_v);
      umma::tma_prefetch_desc(&map_o);
      mbar_arrive_expect_tx(q_full, kTile);
      umma::tma_load_3d(smem + kOffQ, &map_q, 0, q0, bh, q_full);
      umma::tma_load_3d(smem + kOffQ + umma::kSubTileBytes, &map_q, 64, q0, bh, q_full);
      for (int t = 0; t < 2 * nkb; ++t) {        // K_0, V_0, K_1, V_1, ...
        const int slot = t % kSlots, use = t / kSlots;
        if (use > 0 && !mbar_wait_abortable(&empty[slot], (use - 1) & 1, s_abort)) break;
        const CUtensorMap* m = (t & 1) ? &map_v : &map_k;
        unsigned char* dst = smem + kOffRing + slot * kTile;
        mbar_arrive_expect_tx(&full[slot], kTile);
        umma::tma_load_3d(dst, m, 0, (t >> 1) * kQ, bh, &full[slot]);
        umma::tma_load_3d(dst + umma::kSubTileBytes, m, 64, (t >> 1) * kQ, bh, &full[slot]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // narrow heads: only the 16-deep steps that hold real columns of q/k, and an
      // output as wide as v (a multiple of 16 columns)
      const int ksteps = (dk + 15) >> 4;
      constexpr uint32_t idesc_kk = umma::instr_desc_bf16(128, 128, false, false);
      const uint32_t idesc_kn = umma::instr_desc_bf16(128, uint32_t(dv + 15) & ~15u, false, true);
      auto issue_scores = [&](int j) -> bool {
        const int t = 2 * j, slot = t % kSlots;
        if (!mbar_wait_abortable(&full[slot], (t / kSlots) & 1, s_abort)) return false;
        umma::fence_after_sync();
        const uint32_t k_addr = ring_addr + slot * kTile;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          if (ks < ksteps)
            umma::mma_bf16(tmem + kColS, umma::desc_kmajor(q_addr, ks), umma::desc_kmajor(k_addr, ks), idesc_kk,
                           ks > 0);
        umma::mma_commit(s_ready);
        umma::mma_commit(&empty[slot]);
        return true;
      };
      bool ok = mbar_wait_abortable(q_full, 0, s_abort);
      ok = ok && (nkb == 0 || issue_scores(0));
      for (int j = 0; ok && j < nkb; ++j) {
        const int t = 2 * j + 1, slot = t % kSlots;
        if (!mbar_wait_abortable(p_ready, j & 1, s_abort)) break;
        if (!mbar_wait_abortable(&full[slot], (t / kSlots) & 1, s_abort)) break;
        umma::fence_after_sync();
        const uint32_t v_addr = ring_addr + slot * kTile;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_bf16_ts(tmem + kColO, tmem + kColS + ks * 8, umma::desc_mnmajor(v_addr, ks), idesc_kn,
                            (j > 0) || has_state || (ks > 0));
        umma::mma_commit(o_done);
        umma::mma_commit(&empty[slot]);
        // the tensor pipe runs in issue order, so the next scores may overwrite P right away
        if (j + 1 < nkb && !issue_scores(j + 1)) break;
      }
    }
  } else {
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;                  // query row of the block = TMEM lane
    const int tq = q0 + r;                         // global query index
    const uint32_t lane_base = tmem + (uint32_t(q4 * 32) << 16);
    unsigned char* o_tile = smem + kOffO;
    // m_ref: the reference point of the exponentials (units of scale*log2(e)); it
    // follows the running maximum lazily, only when the maximum has moved by more
    // than kLazy, so P stays below 2^kLazy and the O rescale becomes rare.  Any
    // common reference gives the same o = O / l.
    constexpr float kLazy = 8.f;
    constexpr float kLog2e = 1.4426950408889634f;
    const size_t srow = size_t(bh) * Tq + min(tq, Tq - 1);          // this row in the state tensors
    const bool row_in = tq < Tq;
    // a carrier handed in by the caller is (m, l, a) with m in natural-log units
    float m_ref = (has_state && row_in) ? m_in[srow] * kLog2e : -INFINITY;
    float l_run = (has_state && row_in) ? l_in[srow] : 0.f;
    float m_true = m_ref;                                          // the running maximum itself
    uint32_t sv[4][32];                            // this row's 128 scores, then its O row
    const int ncb = (dv + 31) >> 5;                // 32-column groups of O that hold output
    for (int j = 0; j < nkb; ++j) {
      constexpr uint32_t scol = kColS;
      bool ok = mbar_wait_abortable(s_ready, j & 1, s_abort);
      if (!__all_sync(0xffffffffu, ok)) break;
      umma::fence_after_sync();
      const int k0 = j * kQ;
      const bool partial = (causal && k0 + kQ - 1 + key_offset > q0) || (k0 + kQ > Tk);   // uniform over the CTA
#pragma unroll
      for (int cb = 0; cb < 4; ++cb) umma::tmem_ld32(lane_base + scol + cb * 32, sv[cb]);
      umma::tmem_wait_ld();
      // hidden keys (beyond the diagonal or beyond Tk) score -inf: they never win the
      // maximum and exponentiate to exactly 0 (scale > 0 on this path)
      if (partial) {
        const int lim = (causal ? min(tq - key_offset, Tk - 1) : Tk - 1) - k0;   // last visible column of the block
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (cb * 32 + c > lim) sv[cb][c] = 0xff800000u;
      }
      // additive bias (an explicit attention mask): scores here are unscaled, so the bias goes in divided
      // by the scale; -inf hides the key like the causal mask does
      if (BIAS) {
        const float* brow = bias.p + (bh / bias.H) * bias.sb + (bh % bias.H) * bias.sh +
                            (long long)min(tq, Tq - 1) * bias.sq + k0;
        const float unscale = kLog2e / scale_log2e;
        const int nvis = min(kQ, Tk - k0);
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (cb * 32 + c < nvis)
              sv[cb][c] = __float_as_uint(fmaf(__ldg(brow + cb * 32 + c), unscale, __uint_as_float(sv[cb][c])));
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int cb = 0; cb < 4; ++cb)
#pragma unroll
        for (int c = 0; c < 32; ++c) mx[c & 3] = fmaxf(mx[c & 3], __uint_as_float(sv[cb][c]));
      const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2e;
      m_true = fmaxf(m_true, m_blk);
      float alpha = 1.f;
      if (m_blk > m_ref + kLazy || m_ref == -INFINITY) {   // (the second test also covers m_blk = -inf)
        const float m_new = fmaxf(m_ref, m_blk);
        alpha = (m_new == -INFINITY) ? 1.f : ex2(m_ref - m_new);   // 0 on the first visible block
        m_ref = m_new;
      }
      const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t w[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(sv[cb][c]), scale_log2e, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(sv[cb][c + 1]), scale_log2e, neg_m));
          ps[(c >> 1) & 3] += p0 + p1;
          w[c >> 1] = pack_bf16x2(p0, p1);
        }
        umma::tmem_st16(lane_base + scol + cb * 16, w);       // over columns this thread has consumed
      }
      l_run = fmaf(l_run, alpha, (ps[0] + ps[1]) + (ps[2] + ps[3]));
      umma::tmem_wait_st();
      // O <- O * alpha, once the previous block's P.V has landed; skipped by a warp
      // whose 32 rows all kept their reference point
      if (j == 0 && has_state) {
        // O starts from the caller's a (scaled to this block's reference point); columns past dv
        // that the MMA still covers are zero
#pragma unroll
        for (int cb = 0; cb < 4; ++cb) {
          if (cb < ncb) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int f = cb * 32 + c;
              sv[cb][c] = __float_as_uint((row_in && f < dv) ? a_in[srow * dv + f] * alpha : 0.f);
            }
            umma::tmem_st32(lane_base + kColO + cb * 32, sv[cb]);
          }
        }
        umma::tmem_wait_st();
      }
      if (j > 0) {
        ok = mbar_wait_abortable(o_done, (j - 1) & 1, s_abort);
        if (!__all_sync(0xffffffffu, ok)) break;
        umma::fence_after_sync();
        if (!__all_sync(0xffffffffu, alpha == 1.f)) {
#pragma unroll
          for (int cb = 0; cb < 4; ++cb)
            if (cb < ncb) umma::tmem_ld32(lane_base + kColO + cb * 32, sv[cb]);
          umma::tmem_wait_ld();
#pragma unroll
          for (int cb = 0; cb < 4; ++cb) {
            if (cb < ncb) {
#pragma unroll
              for (int c = 0; c < 32; ++c) sv[cb][c] = __float_as_uint(__uint_as_float(sv[cb][c]) * alpha);
              umma::tmem_st32(lane_base + kColO + cb * 32, sv[cb]);
            }
          }
          umma::tmem_wait_st();
        }
      }
      umma::fence_before_sync();
      mbar_arrive(p_ready);
    }
    // read-out: o = O / l  (0/0 = NaN for a row that saw no key, as the reference), or the raw
    // carrier when the caller continues the fold
    bool ok = nkb == 0 || mbar_wait_abortable(o_done, (nkb - 1) & 1, s_abort);
    if (__all_sync(0xffffffffu, ok)) {
      umma::fence_after_sync();
      if (nkb > 0) {
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
          if (cb < ncb) umma::tmem_ld32(lane_base + kColO + cb * 32, sv[cb]);
        umma::tmem_wait_ld();
      } else {
        // no visible key block: the accumulator is the incoming a (or zero)
#pragma unroll
        for (int cb = 0; cb < 4; ++cb)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int f = cb * 32 + c;
            sv[cb][c] = __float_as_uint((has_state && row_in && f < dv) ? a_in[srow * dv + f] : 0.f);
          }
      }
      if (m_out != nullptr) {
        // (m, l, a) relative to the true running maximum, m back in natural-log units
        if (row_in) {
          const float fix = (m_true == -INFINITY) ? 1.f : ex2(m_ref - m_true);
          m_out[srow] = m_true / kLog2e;
          l_out[srow] = l_run * fix;
          float4* dst = reinterpret_cast<float4*>(a_out + srow * dv);
#pragma unroll
          for (int cb = 0; cb < 4; ++cb) {
            if (cb >= ncb) continue;
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              const int f = cb * 32 + c;
              if (f < dv)      // dv is a multiple of 8
                dst[f >> 2] = make_float4(__uint_as_float(sv[cb][c]) * fix, __uint_as_float(sv[cb][c + 1]) * fix,
                                          __uint_as_float(sv[cb][c + 2]) * fix, __uint_as_float(sv[cb][c + 3]) * fix);
            }
          }
        }
      } else {
        const float inv_l = 1.f / l_run;
#pragma unroll
        for (int cb = 0; cb < 4; ++cb) {
          if (cb >= ncb) continue;
          uint32_t w[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2)
            w[c >> 1] = pack_bf16x2(__uint_as_float(sv[cb][c]) * inv_l, __uint_as_float(sv[cb][c + 1]) * inv_l);
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8)
            *reinterpret_cast<uint4*>(o_tile + umma::tile_chunk_offset(r, cb * 32 + c8 * 8)) =
                make_uint4(w[4 * c8], w[4 * c8 + 1], w[4 * c8 + 2], w[4 * c8 + 3]);
        }
        fence_proxy_async_smem();
        // the four softmax warps meet (bounded wait), then one thread stores the tile
        mbar_arrive(wg_sync);
        ok = mbar_wait_abortable(wg_sync, 0, s_abort);
        if (ok && tid == 64) {
          umma::tma_store_3d(&map_o, 0, q0, bh, o_tile);
          if (dv > 64) umma::tma_store_3d(&map_o, 64, q0, bh, o_tile + umma::kSubTileBytes);
          bulk_commit();
          bulk_wait_all<0>();
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
    umma::tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool om_causal_tc_supported(int B, int H, int Tq, int Tk, int dk, int dv, int dtype) {
  // (the caller also requires scale > 0: hidden scores are set to -inf before scaling)
  return dtype == CB2_BF16 && dk >= 8 && dk <= 128 && dk % 8 == 0 && dv >= 8 && dv <= 128 && dv % 8 == 0 &&
         Tq >= 1 && Tk >= 1 && int64_t(B) * H * ((Tq + 127) / 128) < (int64_t(1) << 31);
}

// o == nullptr with m_out/l_out/a_out set: streaming step (raw fp32 carrier out, optional carrier in).
int om_causal_tc_run(const void* q, const void* k, const void* v, void* o, int B, int H, int Tq, int Tk,
                     int dk, int dv, float scale, int causal, int key_offset, const float* m_in,
                     const float* l_in, const float* a_in, float* m_out, float* l_out, float* a_out,
                     const OmBias& bias, int* dev_status, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mo;
  const uint64_t bh = uint64_t(B) * H;
  int rc = umma::make_map_3d(&mq, q, true, dk, Tq, bh, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mk, k, true, dk, Tk, bh, 64, 128, true);
  if (rc == CB2_OK) rc = umma::make_map_3d(&mv, v, true, dv, Tk, bh, 64, 128, true);
  if (rc == CB2_OK) {
    if (o) rc = umma::make_map_3d(&mo, o, true, dv, Tq, bh, 64, 128, true);
    else mo = mq;                                   // unused in the streaming form
  }
  if (rc != CB2_OK) return rc;
  auto* kernel = bias.p ? om_causal_tc_kernel<true> : om_causal_tc_kernel<false>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)) != cudaSuccess)
    return CB2_LAUNCH_FAIL;
  const unsigned grid = unsigned(((Tq + kQ - 1) / kQ) * bh);
  kernel<<<grid, kThreads, kSmemBytes, st>>>(mq, mk, mv, mo, Tq, Tk, dk, dv, int(bh), causal,
                                             scale * 1.4426950408889634f, key_offset, m_in, l_in, a_in, m_out, l_out,
                                             a_out, bias, dev_status);
  CB2_LAUNCH_CHECK();
  return CB2_OK;
}

}  // namespace cb2
