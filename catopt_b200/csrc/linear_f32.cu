// fp32 GEMMs of the folded weight chain: the runtime `linear(input, fused_N)`
// (catopt_torch/torch_bridge.py:1251-1253), the plain `matmul` binding (:1147)
// and the construction-time fold of a chain of Linear weights
// (`IRModule._fold_weight_chains`, torch_bridge.py:2485-2510).
//
// The path promises rel-err <= 1e-5 against the reference's fp32 result, which
// a single TF32 tensor-core pass (10-bit mantissa) cannot give, so these
// kernels multiply and accumulate in full fp32 on the FMA pipes.  A CTA
// computes a 64x64 tile of the output from 16-deep shared-memory slices, each
// thread a 4x4 micro-tile.  When the output has too few tiles to fill 148 SMs
// (the headline case is a 64x512 output), the reduction axis is split across
// grid.z; partial tiles go to caller-provided scratch and a second kernel sums
// them in a fixed order (deterministic) and adds the bias.
#include <cooperative_groups.h>

#include <cstdio>

#include "common.cuh"

namespace cb2 {
// tensor-core path for large row counts (linear_tf32x3.cu)
bool linear_tf32x3_supported(const float* x, const float* w, const float* bias, const float* y, int R,
                             int n_in, int n_out, const void* scratch, size_t scratch_bytes);
size_t linear_tf32x3_scratch_bytes(int n_in, int n_out);
int linear_tf32x3_run(const float* x, const float* w, const float* bias, float* y, int R, int n_in,
                      int n_out, void* scratch, int* dev_status, cudaStream_t st);
int linear_tf32x3_split(const float* w, float* w_split, int n_in, int n_out, cudaStream_t st);
int linear_tf32x3_run_presplit(const float* x, const float* w_split, const float* bias, float* y, int R, int n_in,
                               int n_out, int* dev_status, cudaStream_t st);

namespace {

constexpr int kTile = 64;
constexpr int kSlice = 16;
constexpr int kGemmThreads = 256;

// C[M,N] (+)= A[M,K] . B  with B stored [N,K] (B_NK, the nn.Linear weight
// layout) or [K,N].  k range of this CTA: [z*k_per_split, min(K, ...)).
// Output goes to `out + z*M*N` (z == 0 and a single split: the real output).
template <bool B_NK>
__global__ void __launch_bounds__(kGemmThreads)
sgemm_kernel(const float* __restrict__ A, const float* __restrict__ Bm, float* __restrict__ out,
             int M, int N, int K, int k_per_split) {
  __shared__ __align__(16) float As[kSlice][kTile + 4];
  __shared__ __align__(16) float Bs[kSlice][kTile + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  const int kb = blockIdx.z * k_per_split;
  const int ke = min(K, kb + k_per_split);
  const int tx = tid % 16, ty = tid / 16;  // micro-tile: rows ty*4.., cols tx*4..
  float acc[4][4] = {};

  for (int k0 = kb; k0 < ke; k0 += kSlice) {
    // A slice: 64 rows x 16 k; thread loads 4 consecutive k of one row.
    {
      const int r = tid / 4, kq = (tid % 4) * 4;
      const int gm = m0 + r;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gk = k0 + kq + j;
        As[kq + j][r] = (gm < M && gk < ke) ? A[size_t(gm) * K + gk] : 0.f;
      }
    }
    if (B_NK) {
      const int r = tid / 4, kq = (tid % 4) * 4;
      const int gn = n0 + r;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gk = k0 + kq + j;
        Bs[kq + j][r] = (gn < N && gk < ke) ? Bm[size_t(gn) * K + gk] : 0.f;
      }
    } else {
      const int kk = tid / 16, nq = (tid % 16) * 4;
      const int gk = k0 + kk;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + nq + j;
        Bs[kk][nq + j] = (gn < N && gk < ke) ? Bm[size_t(gk) * N + gn] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kSlice; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a4[4] = {av.x, av.y, av.z, av.w};
      const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* dst = out + size_t(blockIdx.z) * M * N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) dst[size_t(gm) * N + gn] = acc[i][j];
    }
  }
}

// Split-K without a second launch or scratch: the CTAs that share an output
// tile form a thread-block cluster along grid.z (2, 4 or 8 ranks).  Each rank
// accumulates its slice of K into a 64x64 partial tile in its own shared
// memory; after a cluster barrier, rank r sums rows [r*64/S, (r+1)*64/S) of all
// S partial tiles through distributed shared memory in rank order (so the result
// is deterministic), adds the bias and writes y.
constexpr int kSliceC = 64;   // the cluster kernel loads a whole 64-deep slice at once
template <bool B_NK>
__global__ void __launch_bounds__(kGemmThreads)
sgemm_cluster_kernel(const float* __restrict__ A, const float* __restrict__ Bm,
                     const float* __restrict__ bias, float* __restrict__ out, int M, int N, int K,
                     int k_per_split) {
  namespace cg = cooperative_groups;
  // As[k][m], Bs[k][n]; the partial tile later reuses the As storage
  __shared__ __align__(16) float As[kSliceC][kTile + 4];
  __shared__ __align__(16) float Bs[kSliceC][kTile + 4];
  float (*part)[kTile + 4] = As;
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  const int kb = blockIdx.z * k_per_split;
  const int ke = min(K, kb + k_per_split);
  const int tx = tid % 16, ty = tid / 16;
  const bool vec = (K % 4 == 0) && aligned16(A) && aligned16(Bm) && (!B_NK ? (N % 4 == 0) : true);
  float acc[4][4] = {};
  for (int k0 = kb; k0 < ke; k0 += kSliceC) {
    // One exposed memory latency per slice: every load of the slice is issued
    // before anything is consumed.  Rows of 64 k = 16 float4; 256 threads cover
    // 16 rows per pass.
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int r = pass * 16 + tid / 16, kq = (tid % 16) * 4;
      const int gm = m0 + r, gk = k0 + kq;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gm < M) {
        if (vec && gk + 3 < ke) {
          v = *reinterpret_cast<const float4*>(A + size_t(gm) * K + gk);
        } else {
          if (gk < ke) v.x = A[size_t(gm) * K + gk];
          if (gk + 1 < ke) v.y = A[size_t(gm) * K + gk + 1];
          if (gk + 2 < ke) v.z = A[size_t(gm) * K + gk + 2];
          if (gk + 3 < ke) v.w = A[size_t(gm) * K + gk + 3];
        }
      }
      As[kq][r] = v.x; As[kq + 1][r] = v.y; As[kq + 2][r] = v.z; As[kq + 3][r] = v.w;
    }
    if (B_NK) {
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        const int r = pass * 16 + tid / 16, kq = (tid % 16) * 4;
        const int gn = n0 + r, gk = k0 + kq;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gn < N) {
          if (vec && gk + 3 < ke) {
            v = *reinterpret_cast<const float4*>(Bm + size_t(gn) * K + gk);
          } else {
            if (gk < ke) v.x = Bm[size_t(gn) * K + gk];
            if (gk + 1 < ke) v.y = Bm[size_t(gn) * K + gk + 1];
            if (gk + 2 < ke) v.z = Bm[size_t(gn) * K + gk + 2];
            if (gk + 3 < ke) v.w = Bm[size_t(gn) * K + gk + 3];
          }
        }
        Bs[kq][r] = v.x; Bs[kq + 1][r] = v.y; Bs[kq + 2][r] = v.z; Bs[kq + 3][r] = v.w;
      }
    } else {
#pragma unroll
      for (int pass = 0; pass < 4; ++pass) {
        const int kk = pass * 16 + tid / 16, nq = (tid % 16) * 4;
        const int gk = k0 + kk, gn = n0 + nq;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gk < ke) {
          if (vec && gn + 3 < N) {
            v = *reinterpret_cast<const float4*>(Bm + size_t(gk) * N + gn);
          } else {
            if (gn < N) v.x = Bm[size_t(gk) * N + gn];
            if (gn + 1 < N) v.y = Bm[size_t(gk) * N + gn + 1];
            if (gn + 2 < N) v.z = Bm[size_t(gk) * N + gn + 2];
            if (gn + 3 < N) v.w = Bm[size_t(gk) * N + gn + 3];
          }
        }
        *reinterpret_cast<float4*>(&Bs[kk][nq]) = v;
      }
    }
    __syncthreads();
#pragma unroll 16
    for (int kk = 0; kk < kSliceC; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a4[4] = {av.x, av.y, av.z, av.w};
      const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<float4*>(&part[ty * 4 + i][tx * 4]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  cluster.sync();   // every rank's partial tile is complete and visible cluster-wide
  const unsigned S = cluster.num_blocks(), rank = cluster.block_rank();
  const int rows_per = kTile / int(S);
  for (int e = tid; e < rows_per * (kTile / 4); e += kGemmThreads) {
    const int row = int(rank) * rows_per + e / (kTile / 4), c4 = (e % (kTile / 4)) * 4;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (unsigned z = 0; z < S; ++z) {
      const float4 v = *reinterpret_cast<const float4*>(cluster.map_shared_rank(&part[row][c4], z));
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    const int gm = m0 + row;
    if (gm < M) {
      const float o4[4] = {sum.x, sum.y, sum.z, sum.w};
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + c4 + j;
        if (gn < N) out[size_t(gm) * N + gn] = o4[j] + (bias ? bias[gn] : 0.f);
      }
    }
  }
  cluster.sync();   // nobody leaves while a peer may still read its shared memory
}

// y[m,n] = sum_z partial[z][m,n] (+ bias[n]); fixed summation order.
__global__ void splitk_sum_kernel(const float* __restrict__ partial, const float* __restrict__ bias,
                                  float* __restrict__ y, int M, int N, int splits) {
  const size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  const size_t mn = size_t(M) * N;
  if (i >= mn) return;
  float s = 0.f;
  for (int z = 0; z < splits; ++z) s += partial[z * mn + i];
  if (bias) s += bias[i % N];
  y[i] = s;
}

__global__ void add_bias_kernel(const float* __restrict__ bias, float* __restrict__ y, int M, int N) {
  const size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i < size_t(M) * N) y[i] += bias[i % N];
}

// A handful of rows (M <= 64: config 1's x [64, 512]) through a weight in nn.Linear layout.
// The generic tile kernels above stage operands through scalar, conflicting shared-memory
// stores; here both operands stay K-contiguous the way they lie in memory:
//   CTA = 64 rows x 32 output columns x one K slice of a cluster of up to 8 ranks (16 x 8 = 128
//   CTAs for 512 -> 512); 128 threads; a 64-deep slice of x (16 KB) and of w (8 KB) is fetched
//   with every 16-byte load in flight at once and parked in shared memory as rows of 16 float4
//   with the float4 index XORed by (row & 15), so that the micro-tile reads below are conflict
//   free; thread = rows {ty + 16 i} x columns {tx + 8 j} (4 x 4), 64 FMAs per 8 LDS.128;
//   partial tiles are reduced through distributed shared memory in rank order (deterministic).
constexpr int kSmallM = 64, kSmallN = 32, kSmallK = 64, kSmallThreads = 128;

__global__ void __launch_bounds__(kSmallThreads)
sgemm_small_rows_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                        float* __restrict__ out, int M, int N, int K, int k_per_split) {
  namespace cg = cooperative_groups;
  __shared__ __align__(16) float4 As[kSmallM][16];
  __shared__ __align__(16) float4 Bs[kSmallN][16];
  __shared__ __align__(16) float part[kSmallM][kSmallN + 4];
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x, tx = tid % 8, ty = tid / 8;
  const int n0 = blockIdx.x * kSmallN;
  const int kb = blockIdx.z * k_per_split;
  const int ke = min(K, kb + k_per_split);
  float acc[4][4] = {};
  for (int k0 = kb; k0 < ke; k0 += kSmallK) {
    float4 av[8], bv[4];
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int idx = tid + kSmallThreads * p, r = idx >> 4, k4 = idx & 15, gk = k0 + 4 * k4;
      av[p] = (r < M && gk < ke) ? __ldg(reinterpret_cast<const float4*>(A + size_t(r) * K + gk))
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int idx = tid + kSmallThreads * p, r = idx >> 4, k4 = idx & 15, gk = k0 + 4 * k4;
      bv[p] = (n0 + r < N && gk < ke) ? __ldg(reinterpret_cast<const float4*>(W + size_t(n0 + r) * K + gk))
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (k0 > kb) __syncthreads();          // the previous slice has been consumed
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int idx = tid + kSmallThreads * p, r = idx >> 4, k4 = idx & 15;
      As[r][k4 ^ (r & 15)] = av[p];
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int idx = tid + kSmallThreads * p, r = idx >> 4, k4 = idx & 15;
      Bs[r][k4 ^ (r & 15)] = bv[p];
    }
    __syncthreads();
#pragma unroll
    for (int k4 = 0; k4 < 16; ++k4) {
      float4 a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[ty + 16 * i][k4 ^ ty];          // (ty + 16 i) & 15 == ty
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[tx + 8 * j][k4 ^ ((tx + 8 * j) & 15)];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
          acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
          acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
          acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
        }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) part[ty + 16 * i][tx + 8 * j] = acc[i][j];
  cluster.sync();   // every rank's partial tile is complete and visible cluster-wide
  const unsigned S = cluster.num_blocks(), rank = cluster.block_rank();
  const int rows_per = kSmallM / int(S);
  for (int e = tid; e < rows_per * (kSmallN / 4); e += kSmallThreads) {
    const int row = int(rank) * rows_per + e / (kSmallN / 4), c4 = (e % (kSmallN / 4)) * 4;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (unsigned z = 0; z < S; ++z) {
      const float4 v = *reinterpret_cast<const float4*>(cluster.map_shared_rank(&part[row][c4], z));
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    if (row < M) {
      const float o4[4] = {sum.x, sum.y, sum.z, sum.w};
      for (int j = 0; j < 4; ++j) {
        const int gn = n0 + c4 + j;
        if (gn < N) out[size_t(row) * N + gn] = o4[j] + (bias ? bias[gn] : 0.f);
      }
    }
  }
  cluster.sync();   // nobody leaves while a peer may still read its shared memory
}

// 0 = the shape is not this kernel's; otherwise the cluster size (1, 2, 4 or 8 K slices).
int small_rows_splits(const float* A, const float* W, int M, int N, int K) {
  if (M > kSmallM || K % 4 != 0 || K < kSmallK || !aligned16(A) || !aligned16(W)) return 0;
  const int tiles = (N + kSmallN - 1) / kSmallN;
  int s = 1;
  while (s < 8 && tiles * s * 2 <= kNumSMs && K / (s * 2) >= kSmallK) s *= 2;
  return s;
}

int small_rows_run(const float* A, const float* W, const float* bias, float* C, int M, int N, int K, int splits,
                   cudaStream_t st) {
  const int kps = (((K + splits - 1) / splits + 3) / 4) * 4;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((N + kSmallN - 1) / kSmallN, 1, splits);
  cfg.blockDim = dim3(kSmallThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 1;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = splits;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, sgemm_small_rows_kernel, A, W, bias, C, M, N, K, kps) == cudaSuccess ? CB2_OK
                                                                                                      : CB2_LAUNCH_FAIL;
}

// Number of K splits that brings the grid up to about one CTA per SM.
int pick_splits(int M, int N, int K) {
  const int tiles = ((M + kTile - 1) / kTile) * ((N + kTile - 1) / kTile);
  if (tiles >= kNumSMs / 2) return 1;
  int splits = kNumSMs / tiles;
  const int max_by_k = (K + 2 * kSlice - 1) / (2 * kSlice);  // keep >= 32 k per split
  if (splits > max_by_k) splits = max_by_k;
  if (splits > 8) splits = 8;                                // portable cluster size
  return splits < 1 ? 1 : splits;
}

template <bool B_NK>
int gemm(const float* A, const float* Bm, const float* bias, float* C, int M, int N, int K,
         float* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (B_NK) {   // a handful of rows through an nn.Linear weight: the K-contiguous kernel
    const int s = small_rows_splits(A, Bm, M, N, K);
    if (s > 0) {
      if (small_rows_run(A, Bm, bias, C, M, N, K, s, st) == CB2_OK) return CB2_OK;
      (void)cudaGetLastError();   // cluster launch refused: the generic kernels below
    }
  }
  const int splits = pick_splits(M, N, K);
  dim3 grid((N + kTile - 1) / kTile, (M + kTile - 1) / kTile, 1);
  if (splits > 1) {
    // 2/4/8 K-slices: one launch, reduction through distributed shared memory
    int cs = 2;
    while (cs < splits) cs <<= 1;
    const int kps = (((K + cs - 1) / cs + 3) / 4) * 4;   // multiples of 4 keep float4 loads aligned
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid.x, grid.y, cs);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = cs;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, sgemm_cluster_kernel<B_NK>, A, Bm, bias, C, M, N, K, kps);
    if (ce == cudaSuccess) return CB2_OK;
    (void)cudaGetLastError();  // cluster launch refused: fall back to the plain kernels below
    static bool warned = false;
    if (!warned) {
      warned = true;
      fprintf(stderr, "catopt_b200: cluster launch refused (%s); using the two-pass split-K path\n",
              cudaGetErrorString(ce));
    }
    if (scratch && scratch_bytes >= size_t(cs) * M * N * sizeof(float)) {
      grid.z = cs;
      sgemm_kernel<B_NK><<<grid, kGemmThreads, 0, st>>>(A, Bm, scratch, M, N, K, kps);
      CB2_LAUNCH_CHECK();
      const size_t mn = size_t(M) * N;
      splitk_sum_kernel<<<unsigned((mn + 255) / 256), 256, 0, st>>>(scratch, bias, C, M, N, cs);
      CB2_LAUNCH_CHECK();
      return CB2_OK;
    }
    grid.z = 1;
  }
  sgemm_kernel<B_NK><<<grid, kGemmThreads, 0, st>>>(A, Bm, C, M, N, K, K);
  CB2_LAUNCH_CHECK();
  if (bias) {
    const size_t mn = size_t(M) * N;
    add_bias_kernel<<<unsigned((mn + 255) / 256), 256, 0, st>>>(bias, C, M, N);
    CB2_LAUNCH_CHECK();
  }
  return CB2_OK;
}

}  // namespace
}  // namespace cb2

extern "C" size_t cb2_linear_f32_scratch_bytes(int R, int in_features, int out_features) {
  if (R <= 0 || in_features <= 0 || out_features <= 0) return 0;
  // Split-K partials are normally reduced through distributed shared memory
  // (clusters of up to 8 CTAs); the scratch is only used if a cluster launch is
  // refused, and the call works without it.
  // The tensor-core path (large R) needs scratch for w split into its TF32 hi/lo
  // parts; without it the call runs on the FMA pipes.
  if (R >= 256 && in_features % 4 == 0 && out_features % 4 == 0)
    return cb2::linear_tf32x3_scratch_bytes(in_features, out_features);
  const int splits = cb2::pick_splits(R, out_features, in_features);
  return splits > 1 ? size_t(8) * R * out_features * sizeof(float) : 0;
}

extern "C" int cb2_linear_f32(const float* x, const float* w, const float* bias, float* y, int R,
                              int in_features, int out_features, void* scratch,
                              size_t scratch_bytes, int* dev_status, void* stream) {
  if (!x || !w || !y) return CB2_NULL_PTR;
  if (R <= 0 || in_features <= 0 || out_features <= 0) return CB2_BAD_SHAPE;
  if (cb2::linear_tf32x3_supported(x, w, bias, y, R, in_features, out_features, scratch, scratch_bytes))
    return cb2::linear_tf32x3_run(x, w, bias, y, R, in_features, out_features, scratch, dev_status,
                                  static_cast<cudaStream_t>(stream));
  return cb2::gemm<true>(x, w, bias, y, R, out_features, in_features,
                         static_cast<float*>(scratch), scratch_bytes,
                         static_cast<cudaStream_t>(stream));
}

// A weight that never changes (a folded chain) is split into its TF32 parts ONCE:
// cb2_linear_f32_split_weight writes hi then lo ([out, in] fp32 each) into w_split, and
// cb2_linear_f32_presplit runs the tensor-core GEMM on it without re-splitting (3 x the weight
// bytes of traffic saved per call).  Only the shapes the tensor-core path takes.
extern "C" size_t cb2_linear_f32_split_bytes(int in_features, int out_features) {
  if (in_features <= 0 || out_features <= 0 || in_features % 4 || out_features % 4) return 0;
  return cb2::linear_tf32x3_scratch_bytes(in_features, out_features);
}

extern "C" int cb2_linear_f32_split_weight(const float* w, float* w_split, int in_features, int out_features,
                                           void* stream) {
  if (!w || !w_split) return CB2_NULL_PTR;
  if (in_features <= 0 || out_features <= 0 || in_features % 4 || out_features % 4) return CB2_BAD_SHAPE;
  if (!cb2::aligned16(w) || !cb2::aligned16(w_split)) return CB2_BAD_ALIGN;
  return cb2::linear_tf32x3_split(w, w_split, in_features, out_features, static_cast<cudaStream_t>(stream));
}

extern "C" int cb2_linear_f32_presplit(const float* x, const float* w_split, const float* bias, float* y, int R,
                                       int in_features, int out_features, int* dev_status, void* stream) {
  if (!x || !w_split || !y) return CB2_NULL_PTR;
  if (R < 256 || in_features <= 0 || out_features <= 0 || in_features % 4 || out_features % 4) return CB2_BAD_SHAPE;
  if (!cb2::aligned16(x) || !cb2::aligned16(w_split) || !cb2::aligned16(y) || (bias && !cb2::aligned16(bias)))
    return CB2_BAD_ALIGN;
  return cb2::linear_tf32x3_run_presplit(x, w_split, bias, y, R, in_features, out_features, dev_status,
                                         static_cast<cudaStream_t>(stream));
}

extern "C" int cb2_matmul_f32(const float* a, const float* b, float* c, int M, int N, int K,
                              void* stream) {
  if (!a || !b || !c) return CB2_NULL_PTR;
  if (M <= 0 || N <= 0 || K <= 0) return CB2_BAD_SHAPE;
  return cb2::gemm<false>(a, b, nullptr, c, M, N, K, nullptr, 0, static_cast<cudaStream_t>(stream));
}

extern "C" size_t cb2_chain_fold_f32_scratch_bytes(const int* dims, int k) {
  if (!dims || k < 3) return 0;  // k <= 2 needs no intermediate
  size_t rows = 0;
  for (int i = 2; i < k; ++i) rows = dims[i] > int(rows) ? size_t(dims[i]) : rows;
  // two ping-pong intermediates of at most max(dims[2..k-1]) x dims[0] floats
  return 2 * rows * size_t(dims[0]) * sizeof(float);
}

extern "C" int cb2_chain_fold_f32(const float* const* weights, const int* dims, int k, float* out,
                                  void* scratch, size_t scratch_bytes, void* stream) {
  if (!weights || !dims || !out) return CB2_NULL_PTR;
  if (k < 1) return CB2_BAD_SHAPE;
  for (int i = 0; i <= k; ++i)
    if (dims[i] <= 0) return CB2_BAD_SHAPE;
  for (int i = 0; i < k; ++i)
    if (!weights[i]) return CB2_NULL_PTR;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int in0 = dims[0];
  if (k == 1) {
    return cudaMemcpyAsync(out, weights[0], size_t(dims[1]) * in0 * sizeof(float),
                           cudaMemcpyDeviceToDevice, st) == cudaSuccess
               ? CB2_OK
               : CB2_LAUNCH_FAIL;
  }
  const size_t need = cb2_chain_fold_f32_scratch_bytes(dims, k);
  if (need > 0 && (!scratch || scratch_bytes < need)) return CB2_SCRATCH_TOO_SMALL;
  float* ping = static_cast<float*>(scratch);
  float* pong = ping ? ping + need / sizeof(float) / 2 : nullptr;
  // acc_i = W[i] . acc_{i-1},  acc_0 = W[0];  acc_i is [dims[i+1], dims[0]].
  const float* acc = weights[0];
  for (int i = 1; i < k; ++i) {
    float* dst = (i == k - 1) ? out : ((i & 1) ? ping : pong);
    const int rc = cb2::gemm<false>(weights[i], acc, nullptr, dst, dims[i + 1], in0, dims[i],
                                    nullptr, 0, st);
    if (rc != CB2_OK) return rc;
    acc = dst;
  }
  return CB2_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the chain fold.
//
// Some callers cannot allocate device memory at the point where they fold a
// weight chain: a lowering pass that runs inside a region where the caching
// allocator is frozen (for example while another module's CUDA graph is being
// captured on the same device), a host runtime that was handed a fixed memory
// budget at start-up, or a plugin that only receives raw pointers and has no
// allocator of its own.  For them the two ping-pong intermediates of the fold
// live in a file-scope device array that every GPU loading this library holds
// until exit (2 MiB), instead of in caller-provided scratch.
//
// The array's name is only a host-side handle: the device address is looked up
// with cudaGetSymbolAddress, once per device, with that device current, on the
// entry point's first call on that device.  Make that first call outside any
// stream capture.  All calls share the one array, so two calls that overlap on
// the GPU (different streams, or graphs replayed concurrently) race; calls on
// one stream are ordered and safe.  The fold writes every intermediate element
// before it reads it, so nothing has to be cleared between calls.
// ---------------------------------------------------------------------------
namespace cb2 {
namespace {
constexpr size_t kStaticFoldFloats = 2u * 512u * 512u;  // two 512x512 fp32 intermediates
constexpr int kMaxDevices = 64;
}  // namespace
}  // namespace cb2

static __device__ __align__(256) float g_cb2_fold_scratch[cb2::kStaticFoldFloats];
static float* g_cb2_fold_scratch_addr[cb2::kMaxDevices] = {};

extern "C" size_t cb2_chain_fold_f32_noalloc_max_bytes(void) {
  return cb2::kStaticFoldFloats * sizeof(float);
}

extern "C" int cb2_chain_fold_f32_noalloc(const float* const* weights, const int* dims, int k,
                                          float* out, void* stream) {
  if (!weights || !dims || !out) return CB2_NULL_PTR;
  if (k < 1) return CB2_BAD_SHAPE;
  for (int i = 0; i <= k; ++i)
    if (dims[i] <= 0) return CB2_BAD_SHAPE;
  const size_t need = cb2_chain_fold_f32_scratch_bytes(dims, k);
  if (need > cb2::kStaticFoldFloats * sizeof(float)) return CB2_SCRATCH_TOO_SMALL;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= cb2::kMaxDevices) return CB2_LAUNCH_FAIL;
  float* scratch = g_cb2_fold_scratch_addr[dev];
  if (!scratch) {
    // Set-up, once per device: resolve this device's copy of the array.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_cb2_fold_scratch) != cudaSuccess || !p) return CB2_LAUNCH_FAIL;
    scratch = static_cast<float*>(p);
    g_cb2_fold_scratch_addr[dev] = scratch;  // idempotent: a racing thread stores the same value
  }
  return cb2_chain_fold_f32(weights, dims, k, out, scratch, cb2::kStaticFoldFloats * sizeof(float),
                            stream);
}
