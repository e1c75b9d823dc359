/*
 * catopt_b200.h — C ABI of libcatopt_b200.so: sm_100a executors for the
 * lowered-module hot path of catopt (the modules that run after the e-graph
 * has chosen a rewrite).
 *
 * The reference has no foreign-function boundary for this path: its lowered
 * modules are torch.nn.Modules that call eager torch ops.  Each entry point
 * below therefore cites the reference *forward* it replaces (paths relative to
 * the catopt project root).  Conventions shared by every entry point:
 *
 *   - plain pointers and sizes only; every data pointer is DEVICE memory owned
 *     by the caller unless the comment says "host";
 *   - tensors are dense, row-major, in the layouts stated per function;
 *   - the call enqueues work on `stream` (a cudaStream_t passed as void*) and
 *     returns without synchronising; the return value is a CB2_* status that
 *     reports argument and launch errors only;
 *   - no entry point allocates device memory: scratch is caller-provided and
 *     sized by the matching *_scratch_bytes() query;
 *   - kernels that wait on an asynchronous copy bound the wait; when a wait
 *     runs out they store CB2_WAIT_TIMEOUT into `*dev_status` (device int,
 *     may be NULL) and return early instead of spinning.  The status is the
 *     low byte of that word; the decayed-attention kernel puts the source line
 *     of the wait that ran out into the bits above it (status >> 8), as a
 *     diagnostic.
 */
#ifndef CATOPT_B200_H
#define CATOPT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
enum {
  CB2_OK = 0,
  CB2_BAD_SHAPE = 1,         /* a size is zero/negative or violates a stated rule   */
  CB2_BAD_ALIGN = 2,         /* a pointer misses the stated alignment               */
  CB2_UNSUPPORTED_DTYPE = 3, /* dtype code not handled by this entry point          */
  CB2_LAUNCH_FAIL = 4,       /* the CUDA runtime refused the launch                 */
  CB2_WAIT_TIMEOUT = 5,      /* written to *dev_status by a kernel, never returned  */
  CB2_NULL_PTR = 6,          /* a required pointer is NULL                          */
  CB2_SCRATCH_TOO_SMALL = 7  /* scratch_bytes below the *_scratch_bytes() answer    */
};

/* ---- element types ------------------------------------------------------ */
enum { CB2_F32 = 0, CB2_BF16 = 1 };

/* Library version (major*10000 + minor*100 + patch). */
int cb2_version(void);

/* Static string for a status code. */
const char* cb2_status_str(int status);

/* Stream-ordered bounded wait for a device flag (no counterpart in the reference,
 * whose modules never hand work between kernels): a one-thread kernel polls `*flag`
 * (device int, acquire loads) until it is non-zero or `budget_us` microseconds
 * (1 .. 2,000,000) have passed; on expiry it stores CB2_WAIT_TIMEOUT into
 * `*dev_status` and ends — no trap, nothing in flight, the stream and the context
 * stay usable.  It is the hand-off wait of the segmented decayed kernel as a launch
 * of its own: a caller orders a stream behind a flag another stream's kernel sets,
 * and a host-side failure test makes a wait run out against a flag nobody sets. */
int cb2_wait_for_flag(const int* flag, unsigned budget_us, int* dev_status, void* stream);

/* -------------------------------------------------------------------------
 * (d) verify reduction.
 * Replaces the four eager passes of `_verify_pair`
 * (packages/catopt-torch/src/catopt_torch/report.py:128-140):
 *     max_abs = (ref - out).abs().max();  max_ref = ref.abs().max()
 * for `n_seg` independent comparisons of `numel_per_seg` elements each,
 * stored back to back.  The difference is formed the way torch forms it for
 * the tensor dtype (bf16: fp32 subtract, round-to-nearest-even to bf16), so
 * the maxima are bit-identical to the reference's.
 *
 * result: float[n_seg][4] =
 *   { max|ref-out|, max|ref|, 1.0 if any (ref-out) is NaN else 0.0,
 *     1.0 if any ref is NaN else 0.0 }
 * NaNs are excluded from the two maxima and reported through the flags; the
 * host turns a set flag into the NaN that torch's max() would propagate.
 * The call overwrites `result` (no pre-clearing needed).
 * ref/out must be 16-byte aligned; numel_per_seg * sizeof(element) must be a
 * multiple of 16 unless n_seg == 1.
 * ------------------------------------------------------------------------- */
int cb2_verify_reduce(const void* ref, const void* out, int64_t numel_per_seg,
                      int64_t n_seg, int dtype, float* result, void* stream);

/* -------------------------------------------------------------------------
 * (a) folded weight chain.
 * cb2_linear_f32 replaces the `linear` binding on the folded root
 * `linear(input, fused_N)` (packages/catopt-torch/src/catopt_torch/
 * torch_bridge.py:1251-1253):  y[R,out] = x[R,in] . w[out,in]^T  (+ bias[out]
 * when bias != NULL).  fp32 in, fp32 accumulate.
 * Large row counts (R >= 256, in/out multiples of 4, 16-byte aligned pointers)
 * run on the tensor cores with three-pass TF32 splitting; small ones on the
 * fp32 FMA pipes with the reduction axis split across a thread-block cluster.
 * scratch (cb2_linear_f32_scratch_bytes bytes, 16-byte aligned) may be NULL:
 * the tensor-core path needs it (w split into TF32 hi/lo parts once per call)
 * and without it the call runs on the FMA pipes, slower but to the same
 * tolerance; the FMA path uses it only if a cluster launch is refused.
 * ------------------------------------------------------------------------- */
size_t cb2_linear_f32_scratch_bytes(int R, int in_features, int out_features);
int cb2_linear_f32(const float* x, const float* w, const float* bias, float* y,
                   int R, int in_features, int out_features, void* scratch,
                   size_t scratch_bytes, int* dev_status, void* stream);

/* The folded weight of a chain never changes (`_fold_weight_chains` registers it once as
 * `fused_N`, torch_bridge.py:2485-2510), so its TF32 split can be done once as well:
 * cb2_linear_f32_split_weight writes the hi then the lo part ([out,in] fp32 each,
 * cb2_linear_f32_split_bytes bytes, 16-byte aligned) and cb2_linear_f32_presplit is
 * cb2_linear_f32's tensor-core path on that buffer (R >= 256, in/out multiples of 4;
 * other shapes return CB2_BAD_SHAPE and the caller uses cb2_linear_f32). */
size_t cb2_linear_f32_split_bytes(int in_features, int out_features);
int cb2_linear_f32_split_weight(const float* w, float* w_split, int in_features,
                                int out_features, void* stream);
int cb2_linear_f32_presplit(const float* x, const float* w_split, const float* bias, float* y,
                            int R, int in_features, int out_features, int* dev_status,
                            void* stream);

/* cb2_matmul_f32: c[M,N] = a[M,K] . b[K,N], the `matmul` binding
 * (torch_bridge.py:1147) for two dense fp32 matrices. */
int cb2_matmul_f32(const float* a, const float* b, float* c, int M, int N, int K,
                   void* stream);

/* cb2_chain_fold_f32 replaces the matmul arm of `IRModule._fold_weight_chains`
 * (torch_bridge.py:2485-2510) for a chain of k bias-free Linear weights:
 *     out = W[k-1] . ( ... (W[2] . (W[1] . W[0])) )
 * evaluated innermost-first, the association the extracted right-nested term
 * carries.  W[i] has shape [dims[i+1], dims[i]] (nn.Linear's [out,in]);
 * `weights` is a HOST array of k device pointers, `dims` a HOST array of k+1
 * ints; out has shape [dims[k], dims[0]].
 * scratch: two intermediate products, cb2_chain_fold_f32_scratch_bytes(). */
size_t cb2_chain_fold_f32_scratch_bytes(const int* dims, int k);
int cb2_chain_fold_f32(const float* const* weights, const int* dims, int k,
                       float* out, void* scratch, size_t scratch_bytes,
                       void* stream);

/* cb2_chain_fold_f32_noalloc: the same fold for callers that cannot allocate
 * device memory (a lowering pass running while the allocator is frozen, a host
 * runtime with a fixed memory budget, a plugin that only sees raw pointers).
 * It has no counterpart in the reference.  The two intermediates live in a
 * static device array inside the library (cb2_chain_fold_f32_noalloc_max_bytes()
 * = 2 MiB per GPU, held until exit), so the chain must satisfy
 * cb2_chain_fold_f32_scratch_bytes(dims,k) <= that limit (e.g. any chain of
 * Linear maps up to 512x512); larger chains return CB2_SCRATCH_TOO_SMALL.
 * The first call on a device looks up the array's device address and should be
 * made outside any stream capture.  Every call shares the array: calls that
 * overlap on the GPU race, calls on one stream are safe.  Result identical to
 * cb2_chain_fold_f32. */
size_t cb2_chain_fold_f32_noalloc_max_bytes(void);
int cb2_chain_fold_f32_noalloc(const float* const* weights, const int* dims, int k,
                               float* out, void* stream);

/* -------------------------------------------------------------------------
 * (b) chunked decayed attention,  o[t] = sum_{s<=t} gamma_h^(t-s) (q_t.k_s) v_s / scale.
 * Replaces `ChunkedDecayModule._forward_impl`
 * (packages/catopt-carriers/src/catopt_carriers/decayed_lower.py:702-724:
 * `_forward_intra` 609-639 + `_forward_cross` 671-700) for the uniform
 * K-chunk term of `om_decayed_kway_blocks` (om.py:3076-3152), with the O(K^2)
 * pair products replaced by the state carry
 *     O_i = (Q_i K_i^T . D) V_i + diag(g^(r+1)) Q_i S_i ;
 *     S_{i+1} = g^C S_i + (K_i . g^(C-1-r))^T V_i
 * (the recurrence the reference spells in lab/probes/retnet_baseline_probe.py:
 * 77-110).  Only chunk-local exponents appear, so nothing overflows.
 *
 * q,k: [B,H,T,dk]; v,o: [B,H,T,dv]; gamma: float[H] (device, fp32, 0<g<=1);
 * T % chunk == 0.  dtype is the element type of q,k,v,o; products accumulate
 * and the state is carried in fp32.
 * scratch: cb2_decayed_chunk_scratch_bytes() bytes.  fp32 path: per-chunk K^T V
 * products (required).  Tensor-core path (bf16): optional; with it, heads are
 * cut into consecutive segments handled by different CTAs so that the grid
 * fills the GPU's last wave, the fp32 state crossing from one segment to the
 * next through scratch; with fewer heads than half the SMs and 16 chunks or
 * more, the segments run at the same time instead, each from a start state that
 * two small kernels compute up front (K and V are then read twice); without
 * scratch (NULL / too small) one CTA runs each head.
 * The answer is 0 when no cut would help.  Calls that share scratch must not
 * overlap on the GPU.
 * ------------------------------------------------------------------------- */
size_t cb2_decayed_chunk_scratch_bytes(int B, int H, int T, int dk, int dv,
                                       int chunk, int dtype);
/* 1 when cb2_decayed_chunk_fwd runs these sizes on the tensor cores (one launch,
 * state on chip: bf16 with head dims up to 128, or fp32 with head dims up to 64
 * (multiples of 4) and at least 24 (batch, head) units, in three TF32 passes at
 * fp32 accuracy), 0 when it takes one of the other paths (one launch with
 * warp-level TF32 products for a few small chunks, the fp32 FMA pipes otherwise). */
int cb2_decayed_chunk_on_tensor_cores(int B, int H, int T, int dk, int dv,
                                      int chunk, int dtype);
/* How the tensor-core path cuts a call of these sizes into CTAs, given the scratch the size
 * query asks for: 0 one CTA per (batch, head); 1 a head's segments handing their state over
 * in scratch (more heads than SMs: fills the last wave); 2 parallel segments from start
 * states computed by a pre-pass (few heads); 3 two CTAs per head in one launch, the second
 * accumulating the first's state from K and V by itself (a quarter to half as many heads as
 * SMs; no scratch).  -1: the call does not run on the tensor cores.  0, 1 and 3 give the
 * same bits.  fp32 calls on the tensor cores are always 0. */
int cb2_decayed_chunk_plan(int B, int H, int T, int dk, int dv, int chunk, int dtype);
int cb2_decayed_chunk_fwd(const void* q, const void* k, const void* v, void* o,
                          const float* gamma, int B, int H, int T, int dk, int dv,
                          int chunk, float scale, int dtype, void* scratch,
                          size_t scratch_bytes, int* dev_status, void* stream);

/* -------------------------------------------------------------------------
 * (c) diagonal linear recurrence with readout,
 *     h_t[n] = a_t[n] * h_{t-1}[n] + b[n] * x_t ;  y_t = sum_n c[n] * h_t[n].
 * One step is the reference's `applyd(aff_diag(a_t, b*x_t), h)`
 * (torch_bridge.py:1895-1900); the whole sequence replaces the level-batched
 * reduction of `BatchedScanModule._forward_impl`
 * (packages/catopt-carriers/src/catopt_carriers/scan_lower.py:569-698) when
 * every step's readout is wanted (the prefix maps themselves: cb2_diag_prefix_maps).
 *
 * a: [B,T,D,N] (a_bcast_n == 0) or [B,T,D] shared over n (a_bcast_n == 1);
 * x,y: [B,T,D]; b,c: [D,N]; h0 (may be NULL = zeros) and hT (may be NULL):
 * float[B,D,N].  dtype is the element type of a,x,b,c,y; every element is
 * widened to fp32 before any arithmetic, the state and the n-sum stay fp32
 * and y is rounded once.  N must be one of 1,2,4,8,16,32; D*N*sizeof(element)
 * and D*sizeof(element) must be multiples of 16 and all pointers 16-byte
 * aligned.
 * ------------------------------------------------------------------------- */
int cb2_diag_scan_fwd(const void* a, const void* x, const void* b, const void* c,
                      const float* h0, void* y, float* hT, int B, int T, int D,
                      int N, int a_bcast_n, int dtype, int* dev_status,
                      void* stream);

/* Start states of n_seg equal sequence segments of the scan above, so that a call with
 * few (batch, channel-block) units can run as cb2_diag_scan_fwd over the
 * [B*n_seg, T/n_seg, ...] view of the same tensors with h0 = starts (steps compose by
 * the reference's `affd_compose`, torch_bridge.py:1896-1899: a segment's composed map
 * (prod a_t, end state from zero) is taken in one pass over a and x, then
 * S_s = A_(s-1) S_(s-1) + U_(s-1) from S_0 = h0).  a: [B,T,D,N]; x: [B,T,D]; b: [D,N];
 * h0: float[B,D,N] or NULL; starts: float[B,n_seg,D,N]; T % n_seg == 0, N % 4 == 0.
 * scratch: cb2_diag_scan_seg_scratch_bytes() bytes (the segments' maps). */
size_t cb2_diag_scan_seg_scratch_bytes(int B, int D, int N, int n_seg);
int cb2_diag_scan_seg_starts(const void* a, const void* x, const void* b, const float* h0,
                             float* starts, int B, int T, int D, int N, int n_seg, int dtype,
                             void* scratch, size_t scratch_bytes, void* stream);

/* Final state of a diagonal scan straight from its stacked leaf maps:
 *     out = a_root*h + b_root,  (a_root, b_root) = f_0 . f_1 . ... . f_{n-1},
 *     f_j(h) = a_seq[j]*h + b_seq[j],
 * leaves in product order (f_0 = latest step), as `BatchedScanModule.
 * _forward_fused` (scan_lower.py:785-807) hands them to `fused_diag_levels`
 * (packages/catopt-carriers/src/catopt_carriers/scan_fused.py:100-120), whose
 * log2(n) halving levels this replaces by one pass over the leaves (fp32
 * accumulation).  a_seq, b_seq: [n, S] dense; h, out: [S]; element type `dtype`.
 * scratch: cb2_diag_compose_scratch_bytes() bytes (partial maps when n is cut
 * into segments to fill the GPU). */
size_t cb2_diag_compose_scratch_bytes(long long n, long long S, int dtype);
int cb2_diag_compose_apply(const void* a_seq, const void* b_seq, const void* h, void* out,
                           long long n, long long S, int dtype, void* scratch,
                           size_t scratch_bytes, void* stream);

/* The same fold for rows stored in TIME order (row 0 = first step),
 *     out = f_{n-1}( ... f_1( f_0(h) ) ),  f_j(h) = a_rows[j]*h + b_rows[j]:
 * the sequence form `applyd(aff_diag(a, b), h)` folded along the step axis, which
 * the reference's generated scan kernels compute (`_seq_triton_source` and
 * `_seq_binding`, packages/catopt-discovery/src/catopt_discovery/genkernel.py:
 * 1031-1060, 1208-1233).  a_step_stride / b_step_stride: elements between
 * consecutive rows — S, or 0 for one row shared by every step.  Scratch as for
 * cb2_diag_compose_apply. */
int cb2_diag_fold_apply(const void* a_rows, const void* b_rows, const void* h, void* out,
                        long long n, long long S, long long a_step_stride,
                        long long b_step_stride, int dtype, void* scratch,
                        size_t scratch_bytes, void* stream);

/* All prefix maps of rows in time order: pa[t] = a_t * ... * a_0 and pb[t] with
 * h_t = pa[t]*h_0 + pb[t] for every t, the all-prefix scan of
 * `BatchedOmdModule._prefix_scan` (packages/catopt-carriers/src/catopt_carriers/
 * omd_lower.py:771-824: blocks of sqrt(T) serial compose steps, a carry fold over
 * the block totals and one batched compose) in one pass that reads a and b once
 * and writes both maps once.  a_rows, b_rows: [n,S] with the step strides of
 * cb2_diag_fold_apply; pa, pb: [n,S]; element type `dtype`, fp32 running maps.
 * scratch (cb2_diag_prefix_maps_scratch_bytes bytes, 16-byte aligned, may be
 * NULL): when the state alone cannot fill the GPU the steps are cut into
 * segments whose total maps are computed first (in scratch), after which every
 * segment runs from its carry-in; without scratch each thread walks all steps. */
size_t cb2_diag_prefix_maps_scratch_bytes(long long n, long long S, int dtype);
int cb2_diag_prefix_maps(const void* a_rows, const void* b_rows, void* pa, void* pb,
                         long long n, long long S, long long a_step_stride,
                         long long b_step_stride, int dtype, void* scratch,
                         size_t scratch_bytes, void* stream);

/* Every state of the recurrence over rows in time order: out[t] = a_t*out[t-1] + b_t,
 * out[-1] = h.  This is the value of the stacked-map form
 * `applyd(aff_diag(stack(affd_a f_t), stack(affd_b f_t)), h)` with f_t the prefix
 * maps of an unrolled scan, which `gather_applyd_stack`
 * (packages/catopt-carriers/src/catopt_carriers/xcarrier.py:2252-2275, engine
 * 2125-2249) offers for a `stack` of per-step states and the reference's generic
 * module evaluates with one `affd_compose` per step.  a_rows, b_rows: [n,S] with the
 * step strides of cb2_diag_fold_apply; h: [S]; out: [n,S]; fp32 running state;
 * 3 units of traffic per step.  Scratch: cb2_diag_prefix_maps_scratch_bytes (segments
 * when the state alone cannot fill the GPU), may be NULL. */
int cb2_diag_scan_states(const void* a_rows, const void* b_rows, const void* h, void* out,
                         long long n, long long S, long long a_step_stride,
                         long long b_step_stride, int dtype, void* scratch,
                         size_t scratch_bytes, void* stream);

/* -------------------------------------------------------------------------
 * Gated contraction  o[b] = (s[b] * g[gate(b)]) @ v[b] :  the body of the
 * reference's `om_decayed` element, `(s * d) @ v`
 * (packages/catopt-carriers/src/catopt_carriers/om.py:1053-1057), for scores
 * that are already materialised.  Replaces the generated fused-contraction
 * kernel of the reference's codegen tier (`_decayed_triton_source`,
 * `_decayed_binding`, `decayed_triton_bindings`; genkernel.py:1582-1631,
 * 1784-1861, 1903-1925), which this library's sink binds to minted
 * `decayed_<i>_k` ops in its place.
 * s: [nb,T,K]; g: [ng,T,K]; v: [nb,K,dv]; o: [nb,T,dv]; the gate of batch b is
 * g[(b / g_div) % g_mod] (g_mod <= ng): (1,1) one gate for all, (1,H) one per
 * head of a [B,H] batch, (H,B) one per batch entry, (1,nb) one per (b,h).
 * The product s*g is rounded to the tensor dtype as the reference's multiply
 * is, the contraction accumulates in fp32, o is rounded once.
 * bf16 with K, dv multiples of 8, dv <= 128 and 16-byte aligned pointers runs
 * on the tensor cores (cb2_gated_contract_on_tensor_cores() == 1); everything
 * else on the fp32 FMA pipes.  No scratch.
 * ------------------------------------------------------------------------- */
int cb2_gated_contract_on_tensor_cores(long long nb, int T, int K, int dv, int dtype);
int cb2_gated_contract_fwd(const void* s, const void* g, const void* v, void* o,
                           long long nb, long long ng, int T, int K, int dv, int g_div,
                           int g_mod, int dtype, int* dev_status, void* stream);

/* -------------------------------------------------------------------------
 * (b') causal softmax attention through the online-softmax monoid,
 *     o_t = sum_{j<=t} softmax_j(scale * q_t.k_j) v_j      per (batch, head).
 * Replaces `BatchedOMModule._forward_impl` / `StreamingOMModule`
 * (packages/catopt-carriers/src/catopt_carriers/om_lower.py:729-835, 996-1040)
 * on the causal carrier: `om_apply` of an `om_compose` tree of `om_elem` blocks
 * (torch_bridge.py:1974-2006, 1887-1890) whose scores carry the `cmask`
 * strict-upper-triangle mask (om.py:1023-1029; key j hidden from query t when
 * j > t, including the Tq = 1 case that sees only key 0).  Entirely masked
 * blocks contribute 0; a row without any visible key yields NaN (0/0).
 * q: [B,H,Tq,dk]; k: [B,H,Tk,dk]; v: [B,H,Tk,dv]; o: [B,H,Tq,dv]; dk,dv <= 128;
 * `scale` multiplies the scores (the reference folds it into q).  dtype is the
 * element type of all four tensors.  bf16 tensors with dk, dv multiples of 8 run
 * on the tensor cores (bf16 products, fp32 softmax statistics and accumulator);
 * fp32 tensors on the fp32 FMA pipes.
 * ------------------------------------------------------------------------- */
int cb2_om_causal_fwd(const void* q, const void* k, const void* v, void* o, int B,
                      int H, int Tq, int Tk, int dk, int dv, float scale, int dtype,
                      int* dev_status, void* stream);
/* The same executor with the mask as an argument: causal != 0 hides key j from
 * query t when j > t (cb2_om_causal_fwd), causal == 0 is plain softmax
 * attention — the unmasked carrier the reference's sdpa-over-concat law
 * produces (`om_apply(<om_compose tree of om_elem(scores_i, v_i)>)`,
 * catopt_carriers/om_lower.py:729-835). */
int cb2_om_fwd(const void* q, const void* k, const void* v, void* o, int B, int H,
               int Tq, int Tk, int dk, int dv, float scale, int causal, int dtype,
               int* dev_status, void* stream);
/* The same with an explicit attention mask in torch's additive form — the carrier the
 * reference's masked sdpa-over-concat law produces,
 * `om_apply(om_elem(add(scaled scores, attnbias(m)), v))` (catopt_carriers/om.py:1313-1362;
 * `attnbias`, om.py:1036-1050: a float mask is the bias itself, a bool keep-mask is 0 / -inf):
 *     o = softmax(scale * q k^T + bias) v .
 * bias: fp32, element (b, h, t, j) at bias[b*stride_b + h*stride_h + t*stride_q + j] (strides
 * in elements, 0 on a broadcast axis, keys contiguous).  A key with bias -inf is hidden exactly
 * like a causally masked one; a row whose keys are all hidden is NaN, as in the reference. */
int cb2_om_bias_fwd(const void* q, const void* k, const void* v, void* o, const float* bias,
                    long long bias_stride_b, long long bias_stride_h, long long bias_stride_q,
                    int B, int H, int Tq, int Tk, int dk, int dv, float scale, int causal,
                    int dtype, int* dev_status, void* stream);

/* One streaming step of the same monoid: fold a block of keys/values into a
 * running carrier (m, l, a) — `om_step_qk` / `StreamingOMModule.forward_state`
 * (packages/catopt-carriers/src/catopt_carriers/om_lower.py:896-922, 996-1040):
 *     state' = state (+) om_elem(scale * q k^T [masked], v)
 * with `_om_compose`'s rule m' = max(m, m_blk), l' = l e^(m-m') + l_blk e^(m_blk-m'),
 * a likewise (an all-hidden side contributes exactly 0).  The readout
 * `om_apply_state` is a / l.
 * State tensors are fp32 whatever `dtype` is: m, l: float[B,H,Tq]; a: float[B,H,Tq,dv].
 * m_in = l_in = a_in = NULL starts from the identity (-inf, 0, 0); the outputs may
 * alias the inputs.  causal != 0 hides key j of this call from query row t when
 * key_offset + j > t, where key_offset = (keys folded in before this call) -
 * (sequence position of query row 0); it is negative in a decode step whose
 * queries are the newest positions.
 * scratch (cb2_om_step_scratch_bytes bytes, may be NULL): with few queries and
 * many keys (decode) the keys are cut over extra CTAs that each build a partial
 * carrier there, folded in key order afterwards — the monoid is associative.
 * Paths: at most 8 query rows and >= 256 keys: a streaming, memory-bound kernel
 * (needs scratch); bf16 with more rows: the tensor-core kernel, state carried in
 * tensor memory; everything else: the fp32 FMA tile kernel.
 * dev_status: as for the other tensor-core entry points (may be NULL). */
size_t cb2_om_step_scratch_bytes(int B, int H, int Tq, int Tk, int dv);
int cb2_om_step(const void* q, const void* k, const void* v,
                const float* m_in, const float* l_in, const float* a_in,
                float* m_out, float* l_out, float* a_out,
                int B, int H, int Tq, int Tk, int dk, int dv, float scale,
                int causal, int key_offset, int dtype, void* scratch,
                size_t scratch_bytes, int* dev_status, void* stream);
/* The same step for a carrier with an explicit attention mask (see cb2_om_bias_fwd):
 *     state' = state (+) om_elem(scale * q k^T + bias, v)
 * `bias` points at the columns of THIS block's keys: element (b, h, t, j) of the block at
 * bias[b*stride_b + h*stride_h + t*stride_q + j].  Every path of cb2_om_step takes it, the
 * streaming decode kernel (at most 8 query rows, 256 keys or more) included. */
int cb2_om_bias_step(const void* q, const void* k, const void* v, const float* bias,
                     long long bias_stride_b, long long bias_stride_h, long long bias_stride_q,
                     const float* m_in, const float* l_in, const float* a_in,
                     float* m_out, float* l_out, float* a_out,
                     int B, int H, int Tq, int Tk, int dk, int dv, float scale,
                     int causal, int key_offset, int dtype, void* scratch,
                     size_t scratch_bytes, int* dev_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CATOPT_B200_H */
