// Interaction tensor-product kernels: forward message passing and its two backward passes.
//
// One thread block per target atom (forward, edge-gradient pass) or per source atom
// (source-gradient pass), one thread per channel.  The block walks the atom's edge segment
// in batches of kEdgeBatch edges: the channel-independent coupling G_e = K . Y_e of each edge
// is built cooperatively in shared memory, then every thread contracts its own channel with
// fully unrolled generated code (tp_gen.cuh), keeping the per-atom sums in registers.
// The edge lists are sorted, so the sums are segmented reductions: no atomics, and results
// are bit-reproducible from run to run.
#include "kernels.h"
#include "tp_gen.cuh"

namespace tace {

constexpr int kEdgeBatch = 8;

template <typename T, typename TP>
__device__ __forceinline__ void build_G_batch(const T* __restrict__ Y, const int* edge_ids, int nb, T* Gs) {
  // Gs[e][gi] = sum_k gc[k] * Y[edge e][gy[k]]
  const short* gs = TP::gstart();
  const unsigned char* gy = TP::gy();
  const double* gc = TP::gc();
  for (int idx = threadIdx.x; idx < nb * TP::NG; idx += blockDim.x) {
    const int e = idx / TP::NG, gi = idx - e * TP::NG;
    const T* Ye = Y + (long long)edge_ids[e] * TP::D;
    T s = T(0);
    for (int k = gs[gi]; k < gs[gi + 1]; ++k) s += T(gc[k]) * Ye[gy[k]];
    Gs[e * TP::NG + gi] = s;
  }
}

template <typename T, typename TP>
__global__ void __launch_bounds__(256) tp_fwd_kernel(const TPArgs<T> a) {
  const int i = blockIdx.x, c = threadIdx.x, C = a.C;
  __shared__ T Gs[kEdgeBatch * TP::NG];
  __shared__ int eid[kEdgeBatch];
  __shared__ int esrc[kEdgeBatch];
  T acc[TP::NM];
#pragma unroll
  for (int k = 0; k < TP::NM; ++k) acc[k] = T(0);
  const int beg = a.rowptr[i], end = a.rowptr[i + 1];
  for (int e0 = beg; e0 < end; e0 += kEdgeBatch) {
    const int nb = min(kEdgeBatch, end - e0);
    __syncthreads();
    if (threadIdx.x < nb) {
      eid[threadIdx.x] = e0 + threadIdx.x;
      esrc[threadIdx.x] = a.e_src[e0 + threadIdx.x];
    }
    __syncthreads();
    build_G_batch<T, TP>(a.Y, eid, nb, Gs);
    __syncthreads();
    for (int e = 0; e < nb; ++e) {
      const long long s = esrc[e];
      T xv[TP::NX], wv[TP::NP];
#pragma unroll
      for (int k = 0; k < TP::NX; ++k) xv[k] = a.x[(s * TP::NX + k) * C + c];
      const T* We = a.W + (long long)(e0 + e) * TP::NP * C;
#pragma unroll
      for (int p = 0; p < TP::NP; ++p) wv[p] = We[p * C + c];
      TP::template fwd<T>(xv, Gs + e * TP::NG, wv, acc);
    }
  }
  T* Mi = a.M + (long long)i * TP::NM * C;
#pragma unroll
  for (int k = 0; k < TP::NM; ++k) Mi[k * C + c] = acc[k];
}

// Edge-gradient pass: dW[e,p,c] and dY[e,:] for every edge of target atom i.
template <typename T, typename TP>
__global__ void __launch_bounds__(256) tp_bwd_edge_kernel(const TPArgs<T> a) {
  const int i = blockIdx.x, c = threadIdx.x, C = a.C;
  const int nwarp = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ T Gs[kEdgeBatch * TP::NG];
  __shared__ T red[kEdgeBatch * 8 * TP::D];  // [edge][warp][D], up to 8 warps
  __shared__ int eid[kEdgeBatch];
  __shared__ int esrc[kEdgeBatch];
  T gv[TP::NM];
  const T* gMi = a.gM + (long long)i * TP::NM * C;
#pragma unroll
  for (int k = 0; k < TP::NM; ++k) gv[k] = gMi[k * C + c];
  const int beg = a.rowptr[i], end = a.rowptr[i + 1];
  for (int e0 = beg; e0 < end; e0 += kEdgeBatch) {
    const int nb = min(kEdgeBatch, end - e0);
    __syncthreads();
    if (threadIdx.x < nb) {
      eid[threadIdx.x] = e0 + threadIdx.x;
      esrc[threadIdx.x] = a.e_src[e0 + threadIdx.x];
    }
    __syncthreads();
    build_G_batch<T, TP>(a.Y, eid, nb, Gs);
    __syncthreads();
    for (int e = 0; e < nb; ++e) {
      const long long s = esrc[e];
      T xv[TP::NX], wv[TP::NP], dw[TP::NP], dYp[TP::D];
#pragma unroll
      for (int k = 0; k < TP::NX; ++k) xv[k] = a.x[(s * TP::NX + k) * C + c];
      const long long wbase = (long long)(e0 + e) * TP::NP * C;
#pragma unroll
      for (int p = 0; p < TP::NP; ++p) wv[p] = a.W[wbase + p * C + c];
#pragma unroll
      for (int k = 0; k < TP::D; ++k) dYp[k] = T(0);
      TP::template bwdw<T>(xv, gv, Gs + e * TP::NG, wv, dw, dYp);
#pragma unroll
      for (int p = 0; p < TP::NP; ++p) a.dW[wbase + p * C + c] = dw[p];
      // reduce dY over the channels of this warp
#pragma unroll
      for (int k = 0; k < TP::D; ++k) {
        T v = dYp[k];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red[(e * 8 + warp) * TP::D + k] = v;
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nb * TP::D; idx += blockDim.x) {
      const int e = idx / TP::D, k = idx - e * TP::D;
      T v = T(0);
      for (int w = 0; w < nwarp; ++w) v += red[(e * 8 + w) * TP::D + k];
      T* dst = a.dY + (long long)(e0 + e) * TP::D + k;
      *dst = a.accumulate_dY ? (*dst + v) : v;
    }
  }
}

// Source-gradient pass: dx[b] = sum over edges whose source is b.
template <typename T, typename TP>
__global__ void __launch_bounds__(256) tp_bwd_src_kernel(const TPArgs<T> a) {
  const int b = blockIdx.x, c = threadIdx.x, C = a.C;
  __shared__ T Gs[kEdgeBatch * TP::NG];
  __shared__ int eid[kEdgeBatch];
  __shared__ int edst[kEdgeBatch];
  T dx[TP::NX];
#pragma unroll
  for (int k = 0; k < TP::NX; ++k) dx[k] = T(0);
  const int beg = a.rowptr[b], end = a.rowptr[b + 1];
  for (int k0 = beg; k0 < end; k0 += kEdgeBatch) {
    const int nb = min(kEdgeBatch, end - k0);
    __syncthreads();
    if (threadIdx.x < nb) {
      const int e = a.perm[k0 + threadIdx.x];
      eid[threadIdx.x] = e;
      edst[threadIdx.x] = a.e_dst[e];
    }
    __syncthreads();
    build_G_batch<T, TP>(a.Y, eid, nb, Gs);
    __syncthreads();
    for (int e = 0; e < nb; ++e) {
      const long long d = edst[e];
      T gv[TP::NM], wv[TP::NP];
      const T* gMd = a.gM + d * TP::NM * C;
#pragma unroll
      for (int k = 0; k < TP::NM; ++k) gv[k] = gMd[k * C + c];
      const T* We = a.W + (long long)eid[e] * TP::NP * C;
#pragma unroll
      for (int p = 0; p < TP::NP; ++p) wv[p] = We[p * C + c];
      TP::template bwdx<T>(gv, Gs + e * TP::NG, wv, dx);
    }
  }
  T* out = a.dx + (long long)b * TP::NX * C;
#pragma unroll
  for (int k = 0; k < TP::NX; ++k) out[k * C + c] = dx[k];
}

#define TACE_TP_DISPATCH(KERNEL)                                                         \
  if (a.n_seg <= 0) return cudaSuccess;                                                  \
  if (a.C > 256 || (a.C & 31)) return cudaErrorInvalidValue;                             \
  const dim3 grid(a.n_seg), block(a.C);                                                  \
  if (a.L == 1 && a.scalar_src) KERNEL<T, TPX_L1_S><<<grid, block, 0, s>>>(a);           \
  else if (a.L == 1) KERNEL<T, TPX_L1_F><<<grid, block, 0, s>>>(a);                      \
  else if (a.L == 2 && a.scalar_src) KERNEL<T, TPX_L2_S><<<grid, block, 0, s>>>(a);      \
  else if (a.L == 2) KERNEL<T, TPX_L2_F><<<grid, block, 0, s>>>(a);                      \
  else if (a.L == 3 && a.scalar_src) KERNEL<T, TPX_L3_S><<<grid, block, 0, s>>>(a);      \
  else if (a.L == 3) KERNEL<T, TPX_L3_F><<<grid, block, 0, s>>>(a);                      \
  else return cudaErrorInvalidValue;                                                     \
  return cudaGetLastError();

template <typename T> cudaError_t launch_tp_fwd(const TPArgs<T>& a, cudaStream_t s) { TACE_TP_DISPATCH(tp_fwd_kernel) }
template <typename T> cudaError_t launch_tp_bwd_edge(const TPArgs<T>& a, cudaStream_t s) { TACE_TP_DISPATCH(tp_bwd_edge_kernel) }
template <typename T> cudaError_t launch_tp_bwd_src(const TPArgs<T>& a, cudaStream_t s) { TACE_TP_DISPATCH(tp_bwd_src_kernel) }

template cudaError_t launch_tp_fwd<float>(const TPArgs<float>&, cudaStream_t);
template cudaError_t launch_tp_fwd<double>(const TPArgs<double>&, cudaStream_t);
template cudaError_t launch_tp_bwd_edge<float>(const TPArgs<float>&, cudaStream_t);
template cudaError_t launch_tp_bwd_edge<double>(const TPArgs<double>&, cudaStream_t);
template cudaError_t launch_tp_bwd_src<float>(const TPArgs<float>&, cudaStream_t);
template cudaError_t launch_tp_bwd_src<double>(const TPArgs<double>&, cudaStream_t);

}  // namespace tace
