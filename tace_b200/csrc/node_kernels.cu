// Per-atom element-wise kernels: species gather, gate, product basis, read-out, graph sums.
// Feature layout everywhere: [atom][component (l, m)][channel], channel fastest, so a warp
// always touches 32 consecutive channels of one component.
#include <cstdint>
#include "kernels.h"
#include "tp_gen.cuh"

namespace tace {

constexpr double kSigmoidCst = 1.8467055342154763;  // tace/models/mlp.py:43
constexpr double kSiluCst = 1.6791767923989418;     // tace/models/mlp.py:34

template <typename T>
__global__ void fill_zero_kernel(T* p, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) p[i] = T(0);
}
template <typename T>
cudaError_t launch_fill_zero(T* p, long long n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int blocks = (int)(((n + 255) / 256 < 148LL * 16) ? (n + 255) / 256 : 148LL * 16);
  fill_zero_kernel<T><<<blocks, 256, 0, s>>>(p, n);
  return cudaGetLastError();
}

template <typename T>
__global__ void add_inplace_kernel(T* dst, const T* src, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] += src[i];
}
template <typename T>
cudaError_t launch_add_inplace(T* dst, const T* src, long long n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const int blocks = (int)(((n + 255) / 256 < 148LL * 16) ? (n + 255) / 256 : 148LL * 16);
  add_inplace_kernel<T><<<blocks, 256, 0, s>>>(dst, src, n);
  return cudaGetLastError();
}

// V: the row is moved in 16-byte pieces (uint4) when its length and both base addresses allow, else element by element.
template <typename V, bool SCATTER>
__global__ void permute_rows_kernel(const V* __restrict__ src, const int* __restrict__ perm, V* __restrict__ dst, long long n, int row_len) {
  const long long total = n * row_len;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long i = idx / row_len, k = idx - i * row_len;
    const long long j = perm[i];
    if (SCATTER) dst[j * row_len + k] = src[idx]; else dst[idx] = src[j * row_len + k];
  }
}
template <typename T, bool SCATTER>
cudaError_t launch_permute_rows(const T* src, const int* perm, T* dst, long long n, int row_len, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  constexpr int per = 16 / sizeof(T);
  const bool wide = row_len % per == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  const int len = wide ? row_len / per : row_len;
  const long long blocks = (n * len + 255) / 256;
  const unsigned grid = (unsigned)(blocks < 148 * 32 ? blocks : 148 * 32);
  if (wide)
    permute_rows_kernel<uint4, SCATTER><<<grid, 256, 0, s>>>(reinterpret_cast<const uint4*>(src), perm, reinterpret_cast<uint4*>(dst), n, len);
  else
    permute_rows_kernel<T, SCATTER><<<grid, 256, 0, s>>>(src, perm, dst, n, len);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_gather_rows(const T* src, const int* perm, T* dst, long long n, int row_len, cudaStream_t s) {
  return launch_permute_rows<T, false>(src, perm, dst, n, row_len, s);
}
template <typename T>
cudaError_t launch_scatter_rows(const T* src, const int* perm, T* dst, long long n, int row_len, cudaStream_t s) {
  return launch_permute_rows<T, true>(src, perm, dst, n, row_len, s);
}

template <typename T>
__global__ void species_gather_kernel(const T* __restrict__ table, const int* __restrict__ species, T* out, int n, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  out[idx] = table[(long long)species[i] * C + c];
}
template <typename T>
cudaError_t launch_species_gather(const T* table, const int* species, T* out, int n, int C, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const long long tot = (long long)n * C;
  species_gather_kernel<T><<<(unsigned)((tot + 255) / 256), 256, 0, s>>>(table, species, out, n, C);
  return cudaGetLastError();
}

// ---- gate --------------------------------------------------------------------------------------
// Row of Gt per atom, (L + 1 + D) * C long.  m0 != 0 (the reference's gate_m0 = True, nonlinear.py:27-42): [L + 1 gate
// scalars | all D components], every rank scaled by its gate.  m0 == 0 (gate_m0 = False, the e3nn Gate,
// nonlinear.py:43-70): [scalars | L gate scalars | components of ranks >= 1 | unused]; the scalars go through the
// normalised SiLU, rank l >= 1 is scaled by gate l.
// L is a template parameter so that the loops over ranks and components unroll and every load of a thread is in flight
// before its first store.
template <typename T, int L>
__global__ void gate_fwd_kernel(const T* __restrict__ Gt, T* __restrict__ a, int n, int C, int m0) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  constexpr int D = (L + 1) * (L + 1);
  const T* row = Gt + (long long)i * (L + 1 + D) * C;
  T* out = a + (long long)i * D * C;
  T gs[L + 1], v[D];
  if (!m0) {
#pragma unroll
    for (int l = 0; l <= L; ++l) gs[l] = row[l * C + c];
#pragma unroll
    for (int k = 1; k < D; ++k) v[k] = row[(L + k) * C + c];
    out[c] = T(kSiluCst) * silu_(gs[0]);
#pragma unroll
    for (int l = 1; l <= L; ++l) {
      const T gate = T(kSigmoidCst) * sigmoid_(gs[l]);
#pragma unroll
      for (int m = 0; m < 2 * l + 1; ++m) out[(l * l + m) * C + c] = v[l * l + m] * gate;
    }
    return;
  }
#pragma unroll
  for (int l = 0; l <= L; ++l) gs[l] = row[l * C + c];
#pragma unroll
  for (int k = 0; k < D; ++k) v[k] = row[(L + 1 + k) * C + c];
#pragma unroll
  for (int l = 0; l <= L; ++l) {
    const T gate = T(kSigmoidCst) * sigmoid_(gs[l]);
#pragma unroll
    for (int m = 0; m < 2 * l + 1; ++m) out[(l * l + m) * C + c] = v[l * l + m] * gate;
  }
}
template <typename T, int L>
__global__ void gate_bwd_kernel(const T* __restrict__ Gt, const T* __restrict__ ga, T* __restrict__ gGt, int n, int C, int m0) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  constexpr int D = (L + 1) * (L + 1);
  const T* row = Gt + (long long)i * (L + 1 + D) * C;
  const T* g = ga + (long long)i * D * C;
  T* out = gGt + (long long)i * (L + 1 + D) * C;
  T gs[L + 1], v[D], gk[D];
#pragma unroll
  for (int l = 0; l <= L; ++l) gs[l] = row[l * C + c];
#pragma unroll
  for (int k = 0; k < D; ++k) gk[k] = g[k * C + c];
  if (!m0) {
#pragma unroll
    for (int k = 1; k < D; ++k) v[k] = row[(L + k) * C + c];
    out[c] = gk[0] * T(kSiluCst) * silu_grad_(gs[0]);
#pragma unroll
    for (int l = 1; l <= L; ++l) {
      const T sg = sigmoid_(gs[l]);
      const T gate = T(kSigmoidCst) * sg;
      T acc = T(0);
#pragma unroll
      for (int m = 0; m < 2 * l + 1; ++m) {
        const int k = l * l + m;
        acc += gk[k] * v[k];
        out[(L + k) * C + c] = gk[k] * gate;
      }
      out[l * C + c] = acc * T(kSigmoidCst) * sg * (T(1) - sg);
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < D; ++k) v[k] = row[(L + 1 + k) * C + c];
#pragma unroll
  for (int l = 0; l <= L; ++l) {
    const T sg = sigmoid_(gs[l]);
    const T gate = T(kSigmoidCst) * sg;
    T acc = T(0);
#pragma unroll
    for (int m = 0; m < 2 * l + 1; ++m) {
      const int k = l * l + m;
      acc += gk[k] * v[k];
      out[(L + 1 + k) * C + c] = gk[k] * gate;
    }
    out[l * C + c] = acc * T(kSigmoidCst) * sg * (T(1) - sg);
  }
}
template <typename T>
cudaError_t launch_gate_fwd(const T* Gt, T* a, int n, int L, int C, int m0, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const unsigned blocks = (unsigned)(((long long)n * C + 127) / 128);
  if (L == 1) gate_fwd_kernel<T, 1><<<blocks, 128, 0, s>>>(Gt, a, n, C, m0);
  else if (L == 2) gate_fwd_kernel<T, 2><<<blocks, 128, 0, s>>>(Gt, a, n, C, m0);
  else if (L == 3) gate_fwd_kernel<T, 3><<<blocks, 128, 0, s>>>(Gt, a, n, C, m0);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_gate_bwd(const T* Gt, const T* ga, T* gGt, int n, int L, int C, int m0, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const unsigned blocks = (unsigned)(((long long)n * C + 127) / 128);
  if (L == 1) gate_bwd_kernel<T, 1><<<blocks, 128, 0, s>>>(Gt, ga, gGt, n, C, m0);
  else if (L == 2) gate_bwd_kernel<T, 2><<<blocks, 128, 0, s>>>(Gt, ga, gGt, n, C, m0);
  else if (L == 3) gate_bwd_kernel<T, 3><<<blocks, 128, 0, s>>>(Gt, ga, gGt, n, C, m0);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ---- product basis -----------------------------------------------------------------------------
template <typename T, typename PB>
__global__ void __launch_bounds__(128) pb_fwd_kernel(const T* __restrict__ A, T* __restrict__ B2, int n, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  T a[PB::D], b[PB::NB];
  const T* Ai = A + (long long)i * PB::D * C;
#pragma unroll
  for (int k = 0; k < PB::D; ++k) a[k] = Ai[k * C + c];
  PB::template fwd<T>(a, b);
  T* Bi = B2 + (long long)i * PB::NB * C;
#pragma unroll
  for (int k = 0; k < PB::NB; ++k) Bi[k * C + c] = b[k];
}
// gA += d(B2)/dA^T gB2
template <typename T, typename PB>
__global__ void __launch_bounds__(128) pb_bwd_kernel(const T* __restrict__ A, const T* __restrict__ gB2, T* __restrict__ gA, int n, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  T a[PB::D], db[PB::NB], da[PB::D];
  const T* Ai = A + (long long)i * PB::D * C;
  const T* Gi = gB2 + (long long)i * PB::NB * C;
  T* gAi = gA + (long long)i * PB::D * C;
#pragma unroll
  for (int k = 0; k < PB::D; ++k) { a[k] = Ai[k * C + c]; da[k] = gAi[k * C + c]; }
#pragma unroll
  for (int k = 0; k < PB::NB; ++k) db[k] = Gi[k * C + c];
  PB::template bwd<T>(a, db, da);
#pragma unroll
  for (int k = 0; k < PB::D; ++k) gAi[k * C + c] = da[k];
}

#define TACE_PB_DISPATCH(KERNEL, ...)                                                      \
  if (n <= 0) return cudaSuccess;                                                          \
  const unsigned grid = (unsigned)(((long long)n * C + 127) / 128);                        \
  if (L == 1 && Lout < 0) KERNEL<T, PBX_L1_T><<<grid, 128, 0, s>>>(__VA_ARGS__);            \
  else if (L == 1 && Lout == 1) KERNEL<T, PBX_L1_A><<<grid, 128, 0, s>>>(__VA_ARGS__);      \
  else if (L == 2 && Lout < 0) KERNEL<T, PBX_L2_T><<<grid, 128, 0, s>>>(__VA_ARGS__);       \
  else if (L == 2 && Lout == 1) KERNEL<T, PBX_L2_N1><<<grid, 128, 0, s>>>(__VA_ARGS__);     \
  else if (L == 2 && Lout == 2) KERNEL<T, PBX_L2_A><<<grid, 128, 0, s>>>(__VA_ARGS__);      \
  else if (L == 3 && Lout < 0) KERNEL<T, PBX_L3_T><<<grid, 128, 0, s>>>(__VA_ARGS__);       \
  else if (L == 3 && Lout == 1) KERNEL<T, PBX_L3_N1><<<grid, 128, 0, s>>>(__VA_ARGS__);     \
  else if (L == 3 && Lout == 2) KERNEL<T, PBX_L3_N2><<<grid, 128, 0, s>>>(__VA_ARGS__);     \
  else if (L == 3 && Lout == 3) KERNEL<T, PBX_L3_A><<<grid, 128, 0, s>>>(__VA_ARGS__);      \
  else return cudaErrorInvalidValue;                                                       \
  return cudaGetLastError();

template <typename T>
cudaError_t launch_pb_fwd(const T* A, T* B2, int n, int L, int Lout, int C, cudaStream_t s) {
  TACE_PB_DISPATCH(pb_fwd_kernel, A, B2, n, C)
}
template <typename T>
cudaError_t launch_pb_bwd(const T* A, const T* gB2, T* gA, int n, int L, int Lout, int C, cudaStream_t s) {
  TACE_PB_DISPATCH(pb_bwd_kernel, A, gB2, gA, n, C)
}

// ---- gated bilinear product (product_basis.nonlinear = silu_bilineargate, tace/models/_e3nn/prod.py:183-247) ------
// XY holds both factors per (atom, component): channels [0, C) the first, [C, 2C) the second; Zg [n][NP][C] the gate
// pre-activations, one per (path, channel); B2 [n][NB][C] = silu(Zg) * (x (x) [y, 1]) per path.
template <typename T, typename PB>
__global__ void __launch_bounds__(128) pbl_fwd_kernel(const T* __restrict__ XY, const T* __restrict__ Zg, T* __restrict__ B2, int n, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  T x[PB::D], y[PB::D], w[PB::NP], b[PB::NB];
  const T* Xi = XY + (long long)i * PB::D * 2 * C;
#pragma unroll
  for (int k = 0; k < PB::D; ++k) { x[k] = Xi[k * 2 * C + c]; y[k] = Xi[k * 2 * C + C + c]; }
  const T* Zi = Zg + (long long)i * PB::NP * C;
#pragma unroll
  for (int p = 0; p < PB::NP; ++p) w[p] = silu_(Zi[p * C + c]);
  PB::template fwd<T>(x, y, w, b);
  T* Bi = B2 + (long long)i * PB::NB * C;
#pragma unroll
  for (int k = 0; k < PB::NB; ++k) Bi[k * C + c] = b[k];
}
// gXY[.., :C] += dB2/dx^T gB2 (it already holds the gradient that reached x through the first-order coefficients),
// gXY[.., C:] = dB2/dy^T gB2, gZg = silu'(Zg) * dB2/dw^T gB2
template <typename T, typename PB>
__global__ void __launch_bounds__(128) pbl_bwd_kernel(const T* __restrict__ XY, const T* __restrict__ Zg, const T* __restrict__ gB2,
                                                      T* __restrict__ gXY, T* __restrict__ gZg, int n, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  T x[PB::D], y[PB::D], w[PB::NP], db[PB::NB], dx[PB::D], dy[PB::D], dw[PB::NP];
  const T* Xi = XY + (long long)i * PB::D * 2 * C;
  T* gXi = gXY + (long long)i * PB::D * 2 * C;
#pragma unroll
  for (int k = 0; k < PB::D; ++k) { x[k] = Xi[k * 2 * C + c]; y[k] = Xi[k * 2 * C + C + c]; dx[k] = gXi[k * 2 * C + c]; dy[k] = T(0); }
  const T* Zi = Zg + (long long)i * PB::NP * C;
#pragma unroll
  for (int p = 0; p < PB::NP; ++p) w[p] = silu_(Zi[p * C + c]);
  const T* Gi = gB2 + (long long)i * PB::NB * C;
#pragma unroll
  for (int k = 0; k < PB::NB; ++k) db[k] = Gi[k * C + c];
  PB::template bwd<T>(x, y, w, db, dx, dy, dw);
#pragma unroll
  for (int k = 0; k < PB::D; ++k) { gXi[k * 2 * C + c] = dx[k]; gXi[k * 2 * C + C + c] = dy[k]; }
  T* gZi = gZg + (long long)i * PB::NP * C;
#pragma unroll
  for (int p = 0; p < PB::NP; ++p) gZi[p * C + c] = dw[p] * silu_grad_(Zi[p * C + c]);
}
#define TACE_PBL_DISPATCH(KERNEL, ...)                                                     \
  if (n <= 0) return cudaSuccess;                                                          \
  const unsigned grid = (unsigned)(((long long)n * C + 127) / 128);                        \
  if (L == 1 && Lout < 0) KERNEL<T, PBLX_L1_T><<<grid, 128, 0, s>>>(__VA_ARGS__);           \
  else if (L == 1 && Lout == 1) KERNEL<T, PBLX_L1_A><<<grid, 128, 0, s>>>(__VA_ARGS__);     \
  else if (L == 2 && Lout < 0) KERNEL<T, PBLX_L2_T><<<grid, 128, 0, s>>>(__VA_ARGS__);      \
  else if (L == 2 && Lout == 1) KERNEL<T, PBLX_L2_N1><<<grid, 128, 0, s>>>(__VA_ARGS__);    \
  else if (L == 2 && Lout == 2) KERNEL<T, PBLX_L2_A><<<grid, 128, 0, s>>>(__VA_ARGS__);     \
  else if (L == 3 && Lout < 0) KERNEL<T, PBLX_L3_T><<<grid, 128, 0, s>>>(__VA_ARGS__);      \
  else if (L == 3 && Lout == 1) KERNEL<T, PBLX_L3_N1><<<grid, 128, 0, s>>>(__VA_ARGS__);    \
  else if (L == 3 && Lout == 2) KERNEL<T, PBLX_L3_N2><<<grid, 128, 0, s>>>(__VA_ARGS__);    \
  else if (L == 3 && Lout == 3) KERNEL<T, PBLX_L3_A><<<grid, 128, 0, s>>>(__VA_ARGS__);     \
  else return cudaErrorInvalidValue;                                                       \
  return cudaGetLastError();
template <typename T>
cudaError_t launch_pbl_fwd(const T* XY, const T* Zg, T* B2, int n, int L, int Lout, int C, cudaStream_t s) {
  TACE_PBL_DISPATCH(pbl_fwd_kernel, XY, Zg, B2, n, C)
}
template <typename T>
cudaError_t launch_pbl_bwd(const T* XY, const T* Zg, const T* gB2, T* gXY, T* gZg, int n, int L, int Lout, int C, cudaStream_t s) {
  TACE_PBL_DISPATCH(pbl_bwd_kernel, XY, Zg, gB2, gXY, gZg, n, C)
}

// ---- third-order product basis (correlation 3) ---------------------------------------------------
// B3 = (A x A) x A per (atom, channel); B2 is the full second-order basis.  B3 is written / read through the
// channel-strided column of the thread, so only A and B2 live in registers.
template <typename T, typename PB3>
__global__ void __launch_bounds__(128) pb3_fwd_kernel(const T* __restrict__ A, const T* __restrict__ B2, T* __restrict__ B3, int n, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  T a[PB3::D], b2[PB3::NB2];
#pragma unroll
  for (int k = 0; k < PB3::D; ++k) a[k] = A[((long long)i * PB3::D + k) * C + c];
#pragma unroll
  for (int k = 0; k < PB3::NB2; ++k) b2[k] = B2[((long long)i * PB3::NB2 + k) * C + c];
  PB3::template fwd<T>(a, b2, B3 + (long long)i * PB3::NB * C + c, C);
}
// gB2 += d(B3)/dB2^T gB3 (OPERAND 0) or gA += d(B3)/dA^T gB3 (OPERAND 1): two launches keep the register count down
template <typename T, typename PB3, int OPERAND>
__global__ void __launch_bounds__(128) pb3_bwd_kernel(const T* __restrict__ A, const T* __restrict__ B2, const T* __restrict__ gB3,
                                                      T* __restrict__ gB2, T* __restrict__ gA, int n, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)n * C) return;
  const int i = idx / C, c = idx - (long long)i * C;
  const T* g3 = gB3 + (long long)i * PB3::NB * C + c;
  if constexpr (OPERAND == 0) {
    T a[PB3::D], db2[PB3::NB2];
#pragma unroll
    for (int k = 0; k < PB3::D; ++k) a[k] = A[((long long)i * PB3::D + k) * C + c];
    T* out = gB2 + (long long)i * PB3::NB2 * C + c;
#pragma unroll
    for (int k = 0; k < PB3::NB2; ++k) db2[k] = out[(long long)k * C];
    PB3::template bwd_b2<T>(a, g3, C, db2);
#pragma unroll
    for (int k = 0; k < PB3::NB2; ++k) out[(long long)k * C] = db2[k];
  } else {
    T b2[PB3::NB2], da[PB3::D];
#pragma unroll
    for (int k = 0; k < PB3::NB2; ++k) b2[k] = B2[((long long)i * PB3::NB2 + k) * C + c];
    T* out = gA + (long long)i * PB3::D * C + c;
#pragma unroll
    for (int k = 0; k < PB3::D; ++k) da[k] = out[(long long)k * C];
    PB3::template bwd_a<T>(b2, g3, C, da);
#pragma unroll
    for (int k = 0; k < PB3::D; ++k) out[(long long)k * C] = da[k];
  }
}

#define TACE_PB3_DISPATCH(LAUNCH)                                        \
  if (n <= 0) return cudaSuccess;                                        \
  const unsigned grid = (unsigned)(((long long)n * C + 127) / 128);      \
  if (L == 1 && Lout < 0) { LAUNCH(PB3X_L1_T) }                          \
  else if (L == 1 && Lout == 1) { LAUNCH(PB3X_L1_A) }                    \
  else if (L == 2 && Lout < 0) { LAUNCH(PB3X_L2_T) }                     \
  else if (L == 2 && Lout == 1) { LAUNCH(PB3X_L2_N1) }                   \
  else if (L == 2 && Lout == 2) { LAUNCH(PB3X_L2_A) }                    \
  else if (L == 3 && Lout < 0) { LAUNCH(PB3X_L3_T) }                     \
  else if (L == 3 && Lout == 1) { LAUNCH(PB3X_L3_N1) }                   \
  else if (L == 3 && Lout == 2) { LAUNCH(PB3X_L3_N2) }                   \
  else if (L == 3 && Lout == 3) { LAUNCH(PB3X_L3_A) }                    \
  else return cudaErrorInvalidValue;                                     \
  return cudaGetLastError();

template <typename T>
cudaError_t launch_pb3_fwd(const T* A, const T* B2, T* B3, int n, int L, int Lout, int C, cudaStream_t s) {
#define PB3_FWD(P) pb3_fwd_kernel<T, P><<<grid, 128, 0, s>>>(A, B2, B3, n, C);
  TACE_PB3_DISPATCH(PB3_FWD)
#undef PB3_FWD
}
template <typename T>
cudaError_t launch_pb3_bwd(const T* A, const T* B2, const T* gB3, T* gB2, T* gA, int n, int L, int Lout, int C, cudaStream_t s) {
#define PB3_BWD(P) pb3_bwd_kernel<T, P, 0><<<grid, 128, 0, s>>>(A, B2, gB3, gB2, gA, n, C); \
                   pb3_bwd_kernel<T, P, 1><<<grid, 128, 0, s>>>(A, B2, gB3, gB2, gA, n, C);
  TACE_PB3_DISPATCH(PB3_BWD)
#undef PB3_BWD
}

// ---- read-out ------------------------------------------------------------------------------------
// One warp per atom.  Lane j holds the hidden unit r_j (and r_{j+32}): the atom's scalar channels are staged in shared
// memory and broadcast, the weights of head 0 sit in shared memory as [C][H] (r_j: consecutive lanes, consecutive
// words) and, when there is room (with_t), also transposed as [H][C] for the gradient d e / d h_c = sum_j (d e / d r_j)
// W1[c][j], where lanes run over c.  Sums over lanes use a fixed butterfly, so results do not depend on the launch.
template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
template <typename T>
__global__ void readout_kernel(const ReadoutArgs<T> a, int with_t) {
  extern __shared__ unsigned char smem_raw[];
  const int C = a.C, H = a.H, nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* W1s = reinterpret_cast<T*>(smem_raw);       // [C][H], head 0
  T* W1t = W1s + C * H;                           // [H][C], head 0 (with_t)
  T* hrow = W1t + (with_t ? C * H : 0) + warp * C;                        // [C] scalar channels of this warp's atom
  T* dr = W1t + (with_t ? C * H : 0) + nw * C + warp * 64;                // [64] d e / d r_j
  for (int k = threadIdx.x; k < C * H; k += blockDim.x) {
    const T v = a.W1[k];
    W1s[k] = v;
    if (with_t) W1t[(k % H) * C + k / H] = v;
  }
  __syncthreads();
  for (int i = blockIdx.x * nw + warp; i < a.n; i += gridDim.x * nw) {
    const int g = a.atom_graph[i];
    const int f = a.fidelity ? a.fidelity[g] : 0;
    const T* W1 = a.W1 + (long long)f * C * H;  // other heads are read from global memory
    const T* W2 = a.W2 + f * H;
    const T* h = a.h + (long long)i * a.hs;
    __syncwarp();
    for (int c = lane; c < C; c += 32) hrow[c] = h[c];
    __syncwarp();
    T r0 = T(0), r1 = T(0);
    if (f == 0) {
      for (int c = 0; c < C; ++c) {
        const T hc = hrow[c];
        if (lane < H) r0 += hc * W1s[c * H + lane];
        if (lane + 32 < H) r1 += hc * W1s[c * H + lane + 32];
      }
    } else {
      for (int c = 0; c < C; ++c) {
        const T hc = hrow[c];
        if (lane < H) r0 += hc * W1[c * H + lane];
        if (lane + 32 < H) r1 += hc * W1[c * H + lane + 32];
      }
    }
    T e = T(0);
    if (lane < H) { e += T(kSiluCst) * silu_(r0) * W2[lane]; dr[lane] = T(kSiluCst) * silu_grad_(r0) * W2[lane]; }
    if (lane + 32 < H) { e += T(kSiluCst) * silu_(r1) * W2[lane + 32]; dr[lane + 32] = T(kSiluCst) * silu_grad_(r1) * W2[lane + 32]; }
    e = warp_sum(e);
    for (int t = 0; t < a.n_extra; ++t) {
      const T* ht = a.extra_h[t] + (long long)i * a.extra_hs[t];
      T acc = T(0);
      for (int c = lane; c < C; c += 32) acc += ht[c] * a.extra_w[t][f * C + c];
      e += warp_sum(acc);
    }
    if (a.zbl && !a.zbl_after) e += a.zbl[i];
    const int z = f * a.n_el + a.species[i];
    const int n_nodes = a.graph_ptr[g + 1] - a.graph_ptr[g];
    const int n_edges = a.rowptr_dst[a.graph_ptr[g + 1]] - a.rowptr_dst[a.graph_ptr[g]];
    const T sc = (n_nodes == 1 && n_edges == 0) ? T(0) : a.scale[z];
    const T es = (a.zbl && a.zbl_after) ? e * sc + a.zbl[i] : e * sc;
    if (lane == 0) {
      a.e_scaled[i] = es;
      if (a.factor) a.factor[i] = sc;
      if (a.node_energy) a.node_energy[i] = a.e0[z] + es;
    }
    if (a.gh) {
      __syncwarp();  // dr is complete
      T* gh = a.gh + (long long)i * C;
      for (int c = lane; c < C; c += 32) {
        T v = T(0);
        if (f == 0 && with_t) {
          for (int j = 0; j < H; ++j) v += dr[j] * W1t[j * C + c];
        } else {
          for (int j = 0; j < H; ++j) v += dr[j] * W1[c * H + j];
        }
        gh[c] = v * sc;
      }
    }
  }
}
template <typename T>
__global__ void readout_linear_bwd_kernel(T* __restrict__ gh, long long hs, const T* __restrict__ factor, const T* __restrict__ w,
                                          const int* __restrict__ atom_graph, const int* __restrict__ fidelity, long long n, int C) {
  const long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (k >= n * C) return;
  const long long i = k / C;
  const int c = (int)(k - i * C);
  const int f = fidelity ? fidelity[atom_graph[i]] : 0;
  gh[i * hs + c] += factor[i] * w[f * C + c];
}
template <typename T>
cudaError_t launch_readout_linear_bwd(T* gh, long long hs, const T* factor, const T* w, const int* atom_graph, const int* fidelity,
                                      int n, int C, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  readout_linear_bwd_kernel<T><<<(unsigned)(((long long)n * C + 255) / 256), 256, 0, s>>>(gh, hs, factor, w, atom_graph, fidelity, n, C);
  return cudaGetLastError();
}

// dst[i, :width] += src[i, :width] with independent row strides (the identity skip connection)
template <typename T>
__global__ void add_rows_kernel(T* __restrict__ dst, long long dst_stride, const T* __restrict__ src, long long src_stride, long long n,
                                int width) {
  const long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (k >= n * width) return;
  const long long i = k / width;
  const long long c = k - i * width;
  dst[i * dst_stride + c] += src[i * src_stride + c];
}
template <typename T>
cudaError_t launch_add_rows(T* dst, long long dst_stride, const T* src, long long src_stride, long long n, int width, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  add_rows_kernel<T><<<(unsigned)((n * width + 255) / 256), 256, 0, s>>>(dst, dst_stride, src, src_stride, n, width);
  return cudaGetLastError();
}

// ---- rows scaled by the learned edge density ----------------------------------------------------
template <typename T>
__global__ void scale_rows_kernel(T* __restrict__ x, const T* __restrict__ scale, long long n, int width, long long stride) {
  const long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (k >= n * width) return;
  const long long i = k / width;
  x[i * stride + (k - i * width)] *= scale[i];
}
template <typename T>
cudaError_t launch_scale_rows(T* x, const T* scale, long long n, int width, long long stride, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  scale_rows_kernel<T><<<(unsigned)((n * width + 255) / 256), 256, 0, s>>>(x, scale, n, width, stride);
  return cudaGetLastError();
}
template <typename T>
__global__ void density_node_bwd_kernel(T* __restrict__ gx, const T* __restrict__ x, const T* __restrict__ inv, T* __restrict__ gdens,
                                        int width, long long stride) {
  __shared__ T red[256];
  const long long i = blockIdx.x;
  const T iv = inv[i];
  T acc = T(0);
  for (int k = threadIdx.x; k < width; k += blockDim.x) {
    const T g = gx[i * stride + k];
    acc += g * x[i * stride + k];
    gx[i * stride + k] = g * iv;
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) gdens[i] = iv == T(1e9) ? T(0) : -iv * red[0];
}
template <typename T>
cudaError_t launch_density_node_bwd(T* gx, const T* x, const T* inv, T* gdens, long long n, int width, long long stride,
                                    cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  density_node_bwd_kernel<T><<<(unsigned)n, 256, 0, s>>>(gx, x, inv, gdens, width, stride);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_readout(const ReadoutArgs<T>& a, cudaStream_t s) {
  if (a.n <= 0) return cudaSuccess;
  if (a.H > 64) return cudaErrorInvalidValue;
  const size_t w1 = sizeof(T) * (size_t)a.C * a.H;
  int warps = 8;  // fewer warps per block when the weights leave little of the default 48 KB
  while (warps > 1 && w1 + sizeof(T) * (size_t)warps * (a.C + 64) > 48 * 1024) warps >>= 1;
  const size_t per_warp = sizeof(T) * (size_t)warps * (a.C + 64);
  const int with_t = (2 * w1 + per_warp <= 48 * 1024) ? 1 : 0;  // the transposed copy only where it fits as well
  const size_t smem = (with_t ? 2 : 1) * w1 + per_warp;
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  const int blocks = (a.n + warps - 1) / warps;
  readout_kernel<T><<<blocks < 1184 ? blocks : 1184, warps * 32, smem, s>>>(a, with_t);
  return cudaGetLastError();
}

// Energy of every graph: E0 + scaled read-out summed over its atoms.  Graph g is cut into `slices` equal ranges of atoms;
// block (g, j) sums range j in a fixed order (strided partial sums, then a tree), and with more than one slice a second
// launch adds the slice sums in order.  A batch of many small graphs uses one slice; one large system (an MD block) many.
template <typename T>
__global__ void graph_energy_kernel(const T* __restrict__ e_scaled, const T* __restrict__ e0, const int* __restrict__ species,
                                    const int* __restrict__ graph_ptr, const int* __restrict__ fidelity, int n_el, int slices,
                                    T* __restrict__ out) {
  __shared__ T red[256];
  const int g = blockIdx.x, j = blockIdx.y;
  const T* e0f = e0 + (fidelity ? fidelity[g] : 0) * n_el;
  const long long beg = graph_ptr[g], len = graph_ptr[g + 1] - beg;
  const long long lo = beg + len * j / slices, hi = beg + len * (j + 1) / slices;
  T acc = T(0);
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) acc += e0f[species[i]] + e_scaled[i];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[(long long)g * slices + j] = red[0];
}
template <typename T>
__global__ void graph_energy_finish_kernel(const T* __restrict__ partial, int slices, T* __restrict__ energy, int n_graphs) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_graphs) return;
  T acc = T(0);
  for (int j = 0; j < slices; ++j) acc += partial[(long long)g * slices + j];
  energy[g] = acc;
}
template <typename T>
cudaError_t launch_graph_energy(const T* e_scaled, const T* e0, const int* species, const int* graph_ptr, const int* fidelity,
                                int n_el, T* energy, int n_graphs, long long n_atoms, T* partial, cudaStream_t s) {
  if (n_graphs <= 0) return cudaSuccess;
  const int slices = graph_energy_slices(n_atoms, n_graphs);
  if (slices == 1 || !partial) {
    graph_energy_kernel<T><<<dim3(n_graphs, 1), 256, 0, s>>>(e_scaled, e0, species, graph_ptr, fidelity, n_el, 1, energy);
    return cudaGetLastError();
  }
  graph_energy_kernel<T><<<dim3(n_graphs, slices), 256, 0, s>>>(e_scaled, e0, species, graph_ptr, fidelity, n_el, slices, partial);
  graph_energy_finish_kernel<T><<<(n_graphs + 127) / 128, 128, 0, s>>>(partial, slices, energy, n_graphs);
  return cudaGetLastError();
}

#define INST(T)                                                                                               \
  template cudaError_t launch_fill_zero<T>(T*, long long, cudaStream_t);                                      \
  template cudaError_t launch_pb3_fwd<T>(const T*, const T*, T*, int, int, int, int, cudaStream_t);           \
  template cudaError_t launch_pb3_bwd<T>(const T*, const T*, const T*, T*, T*, int, int, int, int, cudaStream_t); \
  template cudaError_t launch_readout_linear_bwd<T>(T*, long long, const T*, const T*, const int*, const int*, int, int, cudaStream_t); \
  template cudaError_t launch_add_inplace<T>(T*, const T*, long long, cudaStream_t);                          \
  template cudaError_t launch_gather_rows<T>(const T*, const int*, T*, long long, int, cudaStream_t);         \
  template cudaError_t launch_scatter_rows<T>(const T*, const int*, T*, long long, int, cudaStream_t);        \
  template cudaError_t launch_species_gather<T>(const T*, const int*, T*, int, int, cudaStream_t);            \
  template cudaError_t launch_gate_fwd<T>(const T*, T*, int, int, int, int, cudaStream_t);                    \
  template cudaError_t launch_gate_bwd<T>(const T*, const T*, T*, int, int, int, int, cudaStream_t);          \
  template cudaError_t launch_pb_fwd<T>(const T*, T*, int, int, int, int, cudaStream_t);                      \
  template cudaError_t launch_pbl_fwd<T>(const T*, const T*, T*, int, int, int, int, cudaStream_t);           \
  template cudaError_t launch_pbl_bwd<T>(const T*, const T*, const T*, T*, T*, int, int, int, int, cudaStream_t); \
  template cudaError_t launch_pb_bwd<T>(const T*, const T*, T*, int, int, int, int, cudaStream_t);            \
  template cudaError_t launch_readout<T>(const ReadoutArgs<T>&, cudaStream_t);                                \
  template cudaError_t launch_add_rows<T>(T*, long long, const T*, long long, long long, int, cudaStream_t);  \
  template cudaError_t launch_scale_rows<T>(T*, const T*, long long, int, long long, cudaStream_t);           \
  template cudaError_t launch_density_node_bwd<T>(T*, const T*, const T*, T*, long long, int, long long, cudaStream_t); \
  template cudaError_t launch_graph_energy<T>(const T*, const T*, const int*, const int*, const int*, int, T*, int, long long, T*, cudaStream_t);
INST(float)
INST(double)
template cudaError_t launch_fill_zero<int>(int*, long long, cudaStream_t);

}  // namespace tace
