// Grouped, irreps-aware GEMM used for every channel-mixing linear layer.
//
//   C[row, :] (+)= A[row, 0:K] @ B[0:K, 0:N] (+ bias)
//
// Rows are (atom, m) pairs of one rank-l block: row r of a problem maps to atom r / q and
// component r % q, and its address is base + atom * s1 + (r % q) * s2, with K (resp. N)
// contiguous.  This lets one kernel read the per-rank slices of the [atom][component][channel]
// feature layout without any transposition.  A launch carries up to kMaxProblems such
// problems (one per rank l) and, for per-species weights (the reference's e3nnElementLinear,
// tace/models/linear.py:377-481), one group per chemical species: atoms are visited through
// a species-sorted permutation and group g uses B + g * b_group_stride.
//
// CUDA-core FP32/FP64 path: 64x64x16 tiles, 256 threads, 4x4 outputs per thread.
#pragma once
#include <cuda_runtime.h>
#include "tace_common.cuh"

namespace tace {

constexpr int kMaxProblems = 4;

template <typename T>
struct GemmProblem {
  const T* A;
  const T* B;
  T* C;
  const T* bias;        // [N] per group, or nullptr
  int q;                // components per atom in this block (2l+1)
  int N, K;
  long long a_s1, a_s2; // atom stride / component stride of A rows
  long long c_s1, c_s2; // same for C rows
  long long b_group_stride, bias_group_stride;
  int accumulate;       // 0: C = ..., 1: C += ...
  const int* tile_ptr;  // grouped launches: [n_groups+1] prefix sum of ceil(atoms_g * q / 64)
};

template <typename T>
struct GemmBatch {
  GemmProblem<T> p[kMaxProblems];
  int n_problems;
  int n_groups;          // 1 unless per-species
  const int* group_ptr;  // [n_groups+1] atom ranges in `atom_map` order, or nullptr (=> all atoms)
  const int* atom_map;   // row position -> atom index of A, or nullptr (identity)
  const int* c_atom_map; // row position -> atom index of C, or nullptr (identity)
  int n_atoms;           // used when group_ptr == nullptr
};

template <typename T>
__global__ void __launch_bounds__(256) gemm_kernel(const GemmBatch<T> batch) {
  constexpr int BM = 64, BN = 64, BK = 16;
  const GemmProblem<T>& P = batch.p[blockIdx.z];
  int group = 0, tile = blockIdx.x;
  int a_begin = 0, a_end = batch.n_atoms;
  if (batch.group_ptr) {
    // blockIdx.x enumerates the (species, row tile) pairs that exist; find ours.
    const int* tp = P.tile_ptr;
    if ((int)blockIdx.x >= tp[batch.n_groups]) return;
    int lo = 0, hi = batch.n_groups;  // largest g with tp[g] <= blockIdx.x
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tp[mid] <= (int)blockIdx.x) lo = mid; else hi = mid;
    }
    group = lo;
    tile = blockIdx.x - tp[lo];
    a_begin = batch.group_ptr[group];
    a_end = batch.group_ptr[group + 1];
  }
  const int q = P.q;
  const int M = (a_end - a_begin) * q;
  const int row0 = tile * BM;
  const int col0 = blockIdx.y * BN;
  if (row0 >= M || col0 >= P.N) return;

  __shared__ T As[BK][BM + 4];
  __shared__ T Bs[BK][BN + 4];
  __shared__ long long a_off[BM];
  __shared__ long long c_off[BM];

  const int tid = threadIdx.x;
  if (tid < BM) {
    const int r = row0 + tid;
    long long ao = -1, co = -1;
    if (r < M) {
      const int pos = a_begin + r / q;
      const int m = r % q;
      const long long a_atom = batch.atom_map ? batch.atom_map[pos] : pos;
      const long long c_atom = batch.c_atom_map ? batch.c_atom_map[pos] : pos;
      ao = a_atom * P.a_s1 + m * P.a_s2;
      co = c_atom * P.c_s1 + m * P.c_s2;
    }
    a_off[tid] = ao;
    c_off[tid] = co;
  }
  __syncthreads();

  const T* __restrict__ Bg = P.B + group * P.b_group_stride;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 thread grid, 4x4 outputs each
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = T(0);

  for (int k0 = 0; k0 < P.K; k0 += BK) {
    // A tile: 64 rows x 16 k  (1024 elements, 4 per thread); k fastest for coalescing
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx / BK, kk = idx % BK;
      const long long ao = a_off[r];
      T v = T(0);
      if (ao >= 0 && k0 + kk < P.K) v = P.A[ao + k0 + kk];
      As[kk][r] = v;
    }
    // B tile: 16 k x 64 cols
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int kk = idx / BN, cc = idx % BN;
      T v = T(0);
      if (k0 + kk < P.K && col0 + cc < P.N) v = Bg[(long long)(k0 + kk) * P.N + col0 + cc];
      Bs[kk][cc] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }

  const T* bias = P.bias ? P.bias + group * P.bias_group_stride : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long co = c_off[ty * 4 + i];
    if (co < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = col0 + tx * 4 + j;
      if (col >= P.N) continue;
      T v = acc[i][j];
      if (bias) v += bias[col];
      if (P.accumulate) v += P.C[co + col];
      P.C[co + col] = v;
    }
  }
}

// n_atoms_total: atoms covered by the launch (all groups together); sizes grid.x.
template <typename T>
inline cudaError_t launch_gemm(const GemmBatch<T>& b, long long n_atoms_total, cudaStream_t stream) {
  int maxN = 0, maxq = 0;
  for (int i = 0; i < b.n_problems; ++i) {
    maxN = b.p[i].N > maxN ? b.p[i].N : maxN;
    maxq = b.p[i].q > maxq ? b.p[i].q : maxq;
  }
  if (n_atoms_total <= 0 || maxN <= 0 || b.n_problems <= 0) return cudaSuccess;
  long long tiles = (n_atoms_total * maxq + 63) / 64;
  if (b.group_ptr) tiles += b.n_groups;  // every group may end with a partial tile
  dim3 grid((unsigned)tiles, (maxN + 63) / 64, b.n_problems);
  gemm_kernel<T><<<grid, 256, 0, stream>>>(b);
  return cudaGetLastError();
}

}  // namespace tace
