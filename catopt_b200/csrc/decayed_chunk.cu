// C-ABI front of the chunked decayed-attention executor: argument checks and
// the choice between the tensor-core kernels (bf16, dk and dv multiples of 8 up to
// 128: state kept on chip, optional scratch for cutting heads into segments;
// fp32 with dk, dv <= 64 and enough heads: three-pass TF32) and the other
// paths: one fused launch with warp-level three-pass TF32 products for a few
// small chunks, three launches on the fp32 FMA pipes with the state in scratch
// otherwise.
#include "common.cuh"

namespace cb2 {
size_t decayed_ffma_scratch_bytes(int B, int H, int T, int dk, int dv, int C);
int decayed_ffma_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B,
                     int H, int T, int dk, int dv, int C, float scale, int dtype, void* scratch,
                     cudaStream_t st);
bool decayed_small_supported(int B, int H, int T, int dk, int dv, int C);
size_t decayed_small_scratch_bytes(int B, int H, int T, int C);
int decayed_small_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B, int H,
                      int T, int dk, int dv, int C, float scale, int dtype, void* scratch, int* dev_status,
                      cudaStream_t st);
bool decayed_tc_supported(int B, int H, int T, int dk, int dv, int C, int dtype);
size_t decayed_tc_scratch_bytes(int B, int H, int T);
int decayed_tc_plan(int B, int H, int T);
int decayed_tc_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B,
                   int H, int T, int dk, int dv, int C, float scale, void* scratch, size_t scratch_bytes,
                   int* dev_status, cudaStream_t st);

bool decayed_tf32_supported(int B, int H, int T, int dk, int dv, int dtype);
int decayed_tf32_run(const void* q, const void* k, const void* v, void* o, const float* gamma, int B, int H,
                     int T, int dk, int dv, float scale, int* dev_status, cudaStream_t st);

namespace {
int check_shape(int B, int H, int T, int dk, int dv, int C) {
  if (B <= 0 || H <= 0 || T <= 0 || dk <= 0 || dv <= 0 || C <= 0) return CB2_BAD_SHAPE;
  if (T % C != 0) return CB2_BAD_SHAPE;
  return CB2_OK;
}
}  // namespace
}  // namespace cb2

extern "C" size_t cb2_decayed_chunk_scratch_bytes(int B, int H, int T, int dk, int dv, int chunk,
                                                  int dtype) {
  if (cb2::check_shape(B, H, T, dk, dv, chunk) != CB2_OK) return 0;
  if (cb2::decayed_tc_supported(B, H, T, dk, dv, chunk, dtype)) return cb2::decayed_tc_scratch_bytes(B, H, T);
  if (cb2::decayed_tf32_supported(B, H, T, dk, dv, dtype)) return 0;
  if (cb2::decayed_small_supported(B, H, T, dk, dv, chunk)) return cb2::decayed_small_scratch_bytes(B, H, T, chunk);
  return cb2::decayed_ffma_scratch_bytes(B, H, T, dk, dv, chunk);
}

extern "C" int cb2_decayed_chunk_on_tensor_cores(int B, int H, int T, int dk, int dv, int chunk, int dtype) {
  return cb2::check_shape(B, H, T, dk, dv, chunk) == CB2_OK &&
                 (cb2::decayed_tc_supported(B, H, T, dk, dv, chunk, dtype) ||
                  cb2::decayed_tf32_supported(B, H, T, dk, dv, dtype))
             ? 1
             : 0;
}

extern "C" int cb2_decayed_chunk_plan(int B, int H, int T, int dk, int dv, int chunk, int dtype) {
  if (!cb2_decayed_chunk_on_tensor_cores(B, H, T, dk, dv, chunk, dtype)) return -1;
  if (!cb2::decayed_tc_supported(B, H, T, dk, dv, chunk, dtype)) return 0;   // fp32: one CTA per head
  return cb2::decayed_tc_plan(B, H, T);
}

extern "C" int cb2_decayed_chunk_fwd(const void* q, const void* k, const void* v, void* o,
                                     const float* gamma, int B, int H, int T, int dk, int dv,
                                     int chunk, float scale, int dtype, void* scratch,
                                     size_t scratch_bytes, int* dev_status, void* stream) {
  if (!q || !k || !v || !o || !gamma) return CB2_NULL_PTR;
  const int rc = cb2::check_shape(B, H, T, dk, dv, chunk);
  if (rc != CB2_OK) return rc;
  if (dtype != CB2_F32 && dtype != CB2_BF16) return CB2_UNSUPPORTED_DTYPE;
  if (!(scale != 0.f)) return CB2_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cb2::decayed_tc_supported(B, H, T, dk, dv, chunk, dtype)) {
    if (!cb2::aligned16(q) || !cb2::aligned16(k) || !cb2::aligned16(v) || !cb2::aligned16(o))
      return CB2_BAD_ALIGN;
    return cb2::decayed_tc_run(q, k, v, o, gamma, B, H, T, dk, dv, chunk, scale, scratch, scratch_bytes,
                               dev_status, st);
  }
  if (cb2::decayed_tf32_supported(B, H, T, dk, dv, dtype)) {
    if (!cb2::aligned16(q) || !cb2::aligned16(k) || !cb2::aligned16(v) || !cb2::aligned16(o))
      return CB2_BAD_ALIGN;
    return cb2::decayed_tf32_run(q, k, v, o, gamma, B, H, T, dk, dv, scale, dev_status, st);
  }
  if (cb2::decayed_small_supported(B, H, T, dk, dv, chunk)) {   // few small chunks: one launch
    if (!scratch || scratch_bytes < cb2::decayed_small_scratch_bytes(B, H, T, chunk)) return CB2_SCRATCH_TOO_SMALL;
    if (reinterpret_cast<uintptr_t>(scratch) & 15u) return CB2_BAD_ALIGN;
    return cb2::decayed_small_run(q, k, v, o, gamma, B, H, T, dk, dv, chunk, scale, dtype, scratch, dev_status, st);
  }
  const size_t need = cb2::decayed_ffma_scratch_bytes(B, H, T, dk, dv, chunk);
  if (!scratch || scratch_bytes < need) return CB2_SCRATCH_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(scratch) & 15u) return CB2_BAD_ALIGN;
  return cb2::decayed_ffma_run(q, k, v, o, gamma, B, H, T, dk, dv, chunk, scale, dtype, scratch, st);
}

extern "C" int cb2_version(void) { return 100; }

extern "C" const char* cb2_status_str(int status) {
  switch (status) {
    case CB2_OK: return "ok";
    case CB2_BAD_SHAPE: return "bad shape";
    case CB2_BAD_ALIGN: return "bad alignment";
    case CB2_UNSUPPORTED_DTYPE: return "unsupported dtype";
    case CB2_LAUNCH_FAIL: return "kernel launch failed";
    case CB2_WAIT_TIMEOUT: return "device wait timed out";
    case CB2_NULL_PTR: return "null pointer";
    case CB2_SCRATCH_TOO_SMALL: return "scratch too small";
    default: return "unknown status";
  }
}
