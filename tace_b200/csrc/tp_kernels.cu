// Interaction tensor-product kernels: forward message passing and its backward pass.
//
// One thread block per target atom, one thread per channel.  The channel-independent coupling
// G_e = K . Y_e of a batch of the block's edges is built in shared memory from the edges' spherical
// harmonics by a few threads running generated straight-line code; then every thread contracts its own channel with fully unrolled generated
// code (tp_gen.cuh) that reads G four entries at a time.
//
// Forward: the output ranks are split into (at most) two groups, one block per (target, group),
// which halves the accumulator registers and doubles the resident warps.
// Backward: one pass per target produces, for every edge, the gradient of the per-edge weights
// (in place over W), of the angular features (reduced over channels with warp shuffles) and of
// the source features (one row per edge, summed per source atom by launch_segment_sum_rows).
// Edge lists are sorted, so every sum is a segmented reduction: no atomics, bit-reproducible.
#include "kernels.h"
#include "tp_gen.cuh"

namespace tace {

constexpr int kEdgeBatch = 8;

// Build the coupling rows G_e = K . Y_e of edges [e0, e0 + nb) in shared memory: the generated row
// builder comes in TP::NPART parts (two per output group); parts [part0, part0 + nparts) are built, one
// thread per (edge, part).
template <typename T, typename TP>
__device__ __forceinline__ void build_G_rows(const T* __restrict__ Y, int e0, int nb, int part0, int nparts, T* Gs) {
  const int t = threadIdx.x;
  if (t < nb * nparts) {
    const int e = t / nparts, part = part0 + (t - e * nparts);
    const T* Ye = Y + (long long)(e0 + e) * TP::D;
    T* Ge = Gs + e * TP::NG;
    if (part == 0) TP::template build_G_part<0, T>(Ye, Ge);
    else if (part == 1) TP::template build_G_part<1, T>(Ye, Ge);
    else if (part == 2) TP::template build_G_part<(TP::NPART > 2 ? 2 : 0), T>(Ye, Ge);
    else TP::template build_G_part<(TP::NPART > 3 ? 3 : 0), T>(Ye, Ge);
  }
}

// ENV: the path weights are multiplied by the per-edge envelope (radial_basis.apply_cutoff = False); a separate
// instantiation so the default kernels carry none of its registers.
template <typename T, typename TP, int GRP, bool ENV>
__global__ void __maxnreg__(128) tp_fwd_kernel(const TPArgs<T> a) {
  constexpr int NMG = GRP == 0 ? TP::NMG0 : TP::NMG1, NPG = GRP == 0 ? TP::NPG0 : TP::NPG1;
  constexpr int P0 = GRP == 0 ? TP::P00 : TP::P01, M0 = GRP == 0 ? TP::M00 : TP::M01;
  const int i = blockIdx.x, c = threadIdx.x, C = a.C;
  __shared__ __align__(16) T Gs[kEdgeBatch * TP::NG];
  __shared__ int esrc[kEdgeBatch];
  T acc[NMG];
#pragma unroll
  for (int k = 0; k < NMG; ++k) acc[k] = T(0);
  const int beg = a.rowptr[i], end = a.rowptr[i + 1];
  for (int e0 = beg; e0 < end; e0 += kEdgeBatch) {
    const int nb = min(kEdgeBatch, end - e0);
    __syncthreads();
    if (threadIdx.x < nb) esrc[threadIdx.x] = a.e_src[e0 + threadIdx.x];
    build_G_rows<T, TP>(a.Y, e0, nb, 2 * GRP, 2, Gs);
    __syncthreads();
    for (int e = 0; e < nb; ++e) {
      const long long s = esrc[e];
      T xv[TP::NX], wv[NPG];
#pragma unroll
      for (int k = 0; k < TP::NX; ++k) xv[k] = a.x[(s * TP::NX + k) * C + c];
      const T* We = a.W + ((long long)(e0 + e - a.e_base) * TP::NP + P0) * C;
#pragma unroll
      for (int p = 0; p < NPG; ++p) wv[p] = We[p * C + c];
      if constexpr (ENV) {
        const T u = a.env[e0 + e];
#pragma unroll
        for (int p = 0; p < NPG; ++p) wv[p] *= u;
      }
      if constexpr (GRP == 0) TP::template fwd0<T>(xv, Gs + e * TP::NG, wv, acc);
      else TP::template fwd1<T>(xv, Gs + e * TP::NG, wv, acc);
    }
  }
  T* Mi = a.M + ((long long)i * TP::NM + M0) * C;
#pragma unroll
  for (int k = 0; k < NMG; ++k) Mi[k * C + c] = acc[k];
}

// Dynamic shared memory: [NM][C] message gradient of the target | G rows | dY partial sums.
template <typename T, typename TP, bool ENV>
__global__ void __maxnreg__(152) tp_bwd_kernel(const TPArgs<T> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int i = blockIdx.x, c = threadIdx.x, C = a.C;
  const int nwarp = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* gMs = reinterpret_cast<T*>(smem_raw);          // [NM][C]
  T* Gs = gMs + TP::NM * C;                          // [kEdgeBatch][NG]
  T* red = Gs + kEdgeBatch * TP::NG;                 // [kEdgeBatch][8 warps][D]
  __shared__ T red_u[kEdgeBatch * 8];                // envelope-gradient partial sums
  __shared__ int esrc[kEdgeBatch];
  const T* gMi = a.gM + (long long)i * TP::NM * C;
  for (int k = 0; k < TP::NM; ++k) gMs[k * C + c] = gMi[k * C + c];  // each thread later reads only its own column
  const int beg = a.rowptr[i], end = a.rowptr[i + 1];
  for (int e0 = beg; e0 < end; e0 += kEdgeBatch) {
    const int nb = min(kEdgeBatch, end - e0);
    __syncthreads();
    if (threadIdx.x < nb) esrc[threadIdx.x] = a.e_src[e0 + threadIdx.x];
    build_G_rows<T, TP>(a.Y, e0, nb, 0, TP::NPART, Gs);
    __syncthreads();
    for (int e = 0; e < nb; ++e) {
      const long long s = esrc[e];
      T xv[TP::NX], wv[TP::NP], dw[TP::NP], dYp[TP::D], dx[TP::NX];
#pragma unroll
      for (int k = 0; k < TP::NX; ++k) { xv[k] = a.x[(s * TP::NX + k) * C + c]; dx[k] = T(0); }
      const long long wbase = (long long)(e0 + e - a.e_base) * TP::NP * C;
#pragma unroll
      for (int p = 0; p < TP::NP; ++p) wv[p] = a.W[wbase + p * C + c];
#pragma unroll
      for (int k = 0; k < TP::D; ++k) dYp[k] = T(0);
      T u = T(1);
      if constexpr (ENV) {
        u = a.env[e0 + e];
#pragma unroll
        for (int p = 0; p < TP::NP; ++p) wv[p] *= u;
      }
      TP::template bwd<T>(xv, gMs + c, C, Gs + e * TP::NG, wv, dw, dYp, dx);
      T du_part = T(0);  // sum_p dw * (unscaled weight) = sum_p dw * wv / u
      if constexpr (ENV) {
#pragma unroll
        for (int p = 0; p < TP::NP; ++p) { du_part += dw[p] * wv[p]; dw[p] *= u; }
        du_part = u > T(0) ? du_part / u : T(0);
      }
#pragma unroll
      for (int p = 0; p < TP::NP; ++p) a.dW[wbase + p * C + c] = dw[p];
      if (a.dxe) {
        T* out = a.dxe + (long long)(e0 + e - a.e_base) * TP::NX * C;
#pragma unroll
        for (int k = 0; k < TP::NX; ++k) out[k * C + c] = dx[k];
      }
#pragma unroll
      for (int k = 0; k < TP::D; ++k) {  // reduce dY over the channels of this warp
        T v = dYp[k];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red[(e * 8 + warp) * TP::D + k] = v;
      }
      if constexpr (ENV) {  // the same reduction for the envelope gradient
        T v = du_part;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red_u[e * 8 + warp] = v;
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
    if (ENV && (int)threadIdx.x < nb) {
      T v = T(0);
      for (int w = 0; w < nwarp; ++w) v += red_u[threadIdx.x * 8 + w];
      T* dst = a.denv + (e0 + threadIdx.x);
      *dst = a.accumulate_denv ? (*dst + v) : v;
    }
  }
}

template <typename T>
__global__ void segment_sum_rows_kernel(const T* __restrict__ dxe, const int* __restrict__ rowptr, const int* __restrict__ perm,
                                        T* __restrict__ gx, int row_len) {
  const int b = blockIdx.x;
  const int beg = rowptr[b], end = rowptr[b + 1];
  for (int k = threadIdx.x; k < row_len; k += blockDim.x) {
    T acc = T(0);
    for (int j = beg; j < end; ++j) acc += dxe[(long long)perm[j] * row_len + k];
    gx[(long long)b * row_len + k] = acc;
  }
}
template <typename T>
cudaError_t launch_segment_sum_rows(const T* dxe, const int* rowptr_src, const int* perm_src, T* gx, int n_atoms, int row_len,
                                    cudaStream_t s) {
  if (n_atoms <= 0) return cudaSuccess;
  segment_sum_rows_kernel<T><<<n_atoms, 256, 0, s>>>(dxe, rowptr_src, perm_src, gx, row_len);
  return cudaGetLastError();
}

template <typename T>
__global__ void chunk_src_sum_kernel(const T* __restrict__ dxe, const int* __restrict__ keys, const int* __restrict__ perm,
                                     long long k0, long long k1, long long key_base, T* __restrict__ gx, int row_len) {
  const long long k = k0 + blockIdx.x;
  const int key = keys[k];
  if (k > k0 && keys[k - 1] == key) return;  // not the head of a run
  long long end = k + 1;
  while (end < k1 && keys[end] == key) ++end;
  T* dst = gx + ((long long)key - key_base) * row_len;
  for (int c = threadIdx.x; c < row_len; c += blockDim.x) {
    T acc = T(0);
    for (long long j = k; j < end; ++j) acc += dxe[((long long)perm[j] - k0) * row_len + c];
    dst[c] += acc;
  }
}
template <typename T>
cudaError_t launch_chunk_src_sum(const T* dxe_chunk, const int* keys, const int* perm, long long k0, long long k1,
                                 long long key_base, T* gx, int row_len, cudaStream_t s) {
  if (k1 <= k0) return cudaSuccess;
  chunk_src_sum_kernel<T><<<(unsigned)(k1 - k0), 128, 0, s>>>(dxe_chunk, keys, perm, k0, k1, key_base, gx, row_len);
  return cudaGetLastError();
}

template <typename T, typename TP>
cudaError_t launch_fwd_t(const TPArgs<T>& a, cudaStream_t s) {
  if (a.env) {
    tp_fwd_kernel<T, TP, 0, true><<<a.n_seg, a.C, 0, s>>>(a);
    if (TP::NGRP > 1) tp_fwd_kernel<T, TP, 1, true><<<a.n_seg, a.C, 0, s>>>(a);
  } else {
    tp_fwd_kernel<T, TP, 0, false><<<a.n_seg, a.C, 0, s>>>(a);
    if (TP::NGRP > 1) tp_fwd_kernel<T, TP, 1, false><<<a.n_seg, a.C, 0, s>>>(a);
  }
  return cudaGetLastError();
}
template <typename T, typename TP>
cudaError_t launch_bwd_t(const TPArgs<T>& a, cudaStream_t s) {
  const size_t smem = sizeof(T) * ((size_t)TP::NM * a.C + kEdgeBatch * TP::NG + kEdgeBatch * 8 * TP::D);
  if (a.env && !a.denv) return cudaErrorInvalidValue;
  static size_t configured[64] = {};  // the attribute belongs to a device: one slot per device ordinal
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidValue;
  if (smem > 48 * 1024 && smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tp_bwd_kernel<T, TP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tp_bwd_kernel<T, TP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[dev] = smem;
  }
  if (a.env) tp_bwd_kernel<T, TP, true><<<a.n_seg, a.C, smem, s>>>(a);
  else tp_bwd_kernel<T, TP, false><<<a.n_seg, a.C, smem, s>>>(a);
  return cudaGetLastError();
}

#define TACE_TP_DISPATCH(FN)                                              \
  if (a.n_seg <= 0) return cudaSuccess;                                   \
  if (a.C > 256 || (a.C & 31)) return cudaErrorInvalidValue;              \
  if (a.L == 1 && a.scalar_src) return FN<T, TPX_L1_S>(a, s);             \
  if (a.L == 1 && a.Lin == 1) return FN<T, TPX_L1_F>(a, s);               \
  if (a.L == 2 && a.scalar_src) return FN<T, TPX_L2_S>(a, s);             \
  if (a.L == 2 && a.Lin == 1) return FN<T, TPX_L2_N1>(a, s);              \
  if (a.L == 2 && a.Lin == 2) return FN<T, TPX_L2_F>(a, s);               \
  if (a.L == 3 && a.scalar_src) return FN<T, TPX_L3_S>(a, s);             \
  if (a.L == 3 && a.Lin == 1) return FN<T, TPX_L3_N1>(a, s);              \
  if (a.L == 3 && a.Lin == 2) return FN<T, TPX_L3_N2>(a, s);              \
  if (a.L == 3 && a.Lin == 3) return FN<T, TPX_L3_F>(a, s);               \
  return cudaErrorInvalidValue;

template <typename T> cudaError_t launch_tp_fwd(const TPArgs<T>& a, cudaStream_t s) { TACE_TP_DISPATCH(launch_fwd_t) }
template <typename T> cudaError_t launch_tp_bwd(const TPArgs<T>& a, cudaStream_t s) { TACE_TP_DISPATCH(launch_bwd_t) }

template cudaError_t launch_tp_fwd<float>(const TPArgs<float>&, cudaStream_t);
template cudaError_t launch_tp_fwd<double>(const TPArgs<double>&, cudaStream_t);
template cudaError_t launch_tp_bwd<float>(const TPArgs<float>&, cudaStream_t);
template cudaError_t launch_tp_bwd<double>(const TPArgs<double>&, cudaStream_t);
template cudaError_t launch_segment_sum_rows<float>(const float*, const int*, const int*, float*, int, int, cudaStream_t);
template cudaError_t launch_segment_sum_rows<double>(const double*, const int*, const int*, double*, int, int, cudaStream_t);
template cudaError_t launch_chunk_src_sum<float>(const float*, const int*, const int*, long long, long long, long long, float*, int, cudaStream_t);
template cudaError_t launch_chunk_src_sum<double>(const double*, const int*, const int*, long long, long long, long long, double*, int, cudaStream_t);

}  // namespace tace
