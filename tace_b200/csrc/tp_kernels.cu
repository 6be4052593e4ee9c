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
#include <cstdint>
#include "kernels.h"
#include "tp_gen.cuh"

namespace tace {

constexpr int kEdgeBatch = 8;

// W consecutive values of T moved as one piece (16 bytes for W = 16 / sizeof(T)).
template <typename T, int W>
struct alignas(sizeof(T) * W) RowVec { T v[W]; };

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

// Partial passes.  Entry `it` of the part of the row list this launch works on (first part: entries [0, *row_split);
// second part: entries [*row_split, n_seg)), or -1 past its end.  The host does not know where the list is split, so every
// launch covers the whole list with blocks of kListRows entries each; blocks beyond the part return at once.  (One entry per
// block would make those idle blocks the majority and their launch cost visible; a fixed number of long-lived blocks would
// keep the exchange's own kernels, which run beside this one, waiting for a free slot.)
constexpr int kListRows = 8;
template <typename T>
__device__ __forceinline__ int tp_row(const TPArgs<T>& a, int it) {
  const int n0 = *a.row_split;
  if (a.row_part == 0) { if (it >= n0) return -1; }
  else { it += n0; if (it >= a.n_seg) return -1; }
  return a.row_ids[it];
}

// ENV: the path weights are multiplied by the per-edge envelope (radial_basis.apply_cutoff = False); a separate
// instantiation so the default kernels carry none of its registers.
// Cubic Hermite interpolation of the tabulated path weights: knot index and the four basis values of one edge
// (and, for the backward pass, the basis derivatives with respect to the edge length).
template <typename T>
struct RtEdge {
  int k;
  T b[4];
  T d[4];
};
template <typename T, bool DERIV>
__device__ __forceinline__ void rt_prepare(const TPArgs<T>& a, T d, RtEdge<T>& r) {
  const T u = d * a.rt_inv_h;
  int k = (int)u;
  k = k < 0 ? 0 : (k > a.rt_K - 1 ? a.rt_K - 1 : k);
  const T t = u - T(k), t2 = t * t, t3 = t2 * t;
  r.k = k;
  r.b[0] = T(2) * t3 - T(3) * t2 + T(1);
  r.b[1] = t3 - T(2) * t2 + t;
  r.b[2] = T(3) * t2 - T(2) * t3;
  r.b[3] = t3 - t2;
  if (DERIV) {
    r.d[0] = (T(6) * t2 - T(6) * t) * a.rt_inv_h;
    r.d[1] = (T(3) * t2 - T(4) * t + T(1)) * a.rt_inv_h;
    r.d[2] = (T(6) * t - T(6) * t2) * a.rt_inv_h;
    r.d[3] = (T(3) * t2 - T(2) * t) * a.rt_inv_h;
  }
}
// One table entry = (W_k, h W'_k, W_{k+1}, h W'_{k+1}) of a (path, channel) pair for the interval [d_k, d_{k+1}]: the
// four numbers the interpolation needs, in one 16-byte load.
template <typename T>
__device__ __forceinline__ void rt_load(const T* p, T& v0, T& m0, T& v1, T& m1) { v0 = p[0]; m0 = p[1]; v1 = p[2]; m1 = p[3]; }
template <>
__device__ __forceinline__ void rt_load<float>(const float* p, float& v0, float& m0, float& v1, float& m1) {
  const float4 q = __ldg(reinterpret_cast<const float4*>(p));
  v0 = q.x; m0 = q.y; v1 = q.z; m1 = q.w;
}

// RT: path weights interpolated from the table a.rtab instead of read from a.W.
// Messages of target atom i (output group GRP); Gs, esrc, rts: shared memory of the block.
template <typename T, typename TP, int GRP, bool ENV, bool RT>
__device__ __forceinline__ void tp_fwd_row(const TPArgs<T>& a, int i, T* Gs, int* esrc, RtEdge<T>* rts) {
  constexpr int NMG = GRP == 0 ? TP::NMG0 : TP::NMG1, NPG = GRP == 0 ? TP::NPG0 : TP::NPG1;
  constexpr int P0 = GRP == 0 ? TP::P00 : TP::P01, M0 = GRP == 0 ? TP::M00 : TP::M01;
  const int c = threadIdx.x, C = a.C;
  const int rt_first = blockDim.x > 32 ? 32 : 0;  // the second warp (when there is one) prepares the interpolation
  T acc[NMG];
#pragma unroll
  for (int k = 0; k < NMG; ++k) acc[k] = T(0);
  const int beg = a.rowptr[i], end = a.rowptr[i + 1];
  for (int e0 = beg; e0 < end; e0 += kEdgeBatch) {
    const int nb = min(kEdgeBatch, end - e0);
    __syncthreads();
    if (threadIdx.x < nb) esrc[threadIdx.x] = a.e_src[e0 + threadIdx.x];
    if (RT && (int)threadIdx.x >= rt_first && (int)threadIdx.x < rt_first + nb)
      rt_prepare<T, false>(a, a.dlen[e0 + threadIdx.x - rt_first], rts[threadIdx.x - rt_first]);
    build_G_rows<T, TP>(a.Y, e0, nb, 2 * GRP, 2, Gs);
    __syncthreads();
    for (int e = 0; e < nb; ++e) {
      const long long s = esrc[e];
      T xv[TP::NX], wv[NPG];
#pragma unroll
      for (int k = 0; k < TP::NX; ++k) xv[k] = a.x[(s * TP::NX + k) * C + c];
      if constexpr (RT) {
        const T* r0 = a.rtab + ((long long)rts[e].k * TP::NP * C + (long long)P0 * C + c) * 4;
        const T b0 = rts[e].b[0], b1 = rts[e].b[1], b2 = rts[e].b[2], b3 = rts[e].b[3];
#pragma unroll
        for (int p = 0; p < NPG; ++p) {
          T v0, m0, v1, m1;
          rt_load<T>(r0 + (long long)p * C * 4, v0, m0, v1, m1);
          wv[p] = b0 * v0 + b1 * m0 + b2 * v1 + b3 * m1;
        }
      } else {
        const T* We = a.W + ((long long)(e0 + e - a.e_base) * TP::NP + P0) * C;
#pragma unroll
        for (int p = 0; p < NPG; ++p) wv[p] = We[p * C + c];
      }
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
// LIST: block b works on kListRows entries of the row list of a partial pass (tp_row); otherwise block i = target i.
template <typename T, typename TP, int GRP, bool ENV, bool RT, bool LIST>
__global__ void __maxnreg__(128) tp_fwd_kernel(const TPArgs<T> a) {
  __shared__ __align__(16) T Gs[kEdgeBatch * TP::NG];
  __shared__ int esrc[kEdgeBatch];
  __shared__ RtEdge<T> rts[RT ? kEdgeBatch : 1];
  if constexpr (LIST) {
    for (int it = blockIdx.x * kListRows; it < (blockIdx.x + 1) * kListRows; ++it) {
      const int i = tp_row(a, it);
      if (i < 0) break;
      tp_fwd_row<T, TP, GRP, ENV, RT>(a, i, Gs, esrc, rts);
    }
  } else {
    tp_fwd_row<T, TP, GRP, ENV, RT>(a, blockIdx.x, Gs, esrc, rts);
  }
}

// Path weights of one (edge, channel) in the backward pass, interpolated from the table when their path comes up and
// forgotten when it is done: get<p>() turns the entry fetched one path ahead into the weight (and keeps dW_p/dd), asks for
// the entry of path p + 1, and put<p>() folds dE/dW_p into the two per-edge sums that are all the pass keeps of it,
// dE/d(length) += dE/dW_p dW_p/dd and, with an envelope u on the weights, dE/du += dE/dW_p W_p.  Twenty-three weights
// and as many gradients never sit in registers together, and every table entry is read once.
template <typename T, typename TP, bool ENV>
struct RtBwdWeights {
  const T* row;       // table entries of this edge's interval, this thread's channel: path p at row + p * stride
  long long stride;   // 4 * C
  T b0, b1, b2, b3, d0, d1, d2, d3, u;
  T v0, m0, v1, m1;   // entry of the next path
  T w_now, wd_now;    // weight and length derivative of the path in flight
  T dr, du;
  __device__ __forceinline__ void start() {
    dr = T(0); du = T(0);
    rt_load<T>(row, v0, m0, v1, m1);
  }
  template <int P> __device__ __forceinline__ T get() {
    w_now = b0 * v0 + b1 * m0 + b2 * v1 + b3 * m1;
    wd_now = d0 * v0 + d1 * m0 + d2 * v1 + d3 * m1;
    if (P + 1 < TP::NP) rt_load<T>(row + (long long)(P + 1) * stride, v0, m0, v1, m1);
    return ENV ? w_now * u : w_now;
  }
  template <int P> __device__ __forceinline__ void put(T dwv) {
    if (ENV) { du += dwv * w_now; dr += dwv * u * wd_now; }
    else dr += dwv * wd_now;
  }
};

// The same for path weights held in memory (W[edge][path][channel]): each weight is loaded one path ahead of its use
// and its gradient stored as soon as it is known.
template <typename T, typename TP, bool ENV>
struct ArrayBwdWeights {
  const T* W;   // this edge's weights, this thread's channel: path p at W[p * C]
  T* dW;
  int C;
  T u, next, w_now, du;
  __device__ __forceinline__ void start() { du = T(0); next = W[0]; }
  template <int P> __device__ __forceinline__ T get() {
    w_now = next;
    if (P + 1 < TP::NP) next = W[(P + 1) * C];
    return ENV ? w_now * u : w_now;
  }
  template <int P> __device__ __forceinline__ void put(T dwv) {
    if (ENV) { du += dwv * w_now; dW[P * C] = dwv * u; }
    else dW[P * C] = dwv;
  }
};

// Sums of N per-lane values over the 32 lanes of a warp, all N at once: in each of the first steps a lane hands one half
// of the values it still holds to its partner (lane ^ 16, ^ 8, ...) and adds the partner's copy of the other half, so the
// number of values per lane halves with every exchange, instead of N separate five-step butterflies.  Afterwards every
// lane holds the complete sum of one value; `k` is its index on the one lane that is to store it and N on all others
// (copies of the same sum, padding).  About 4 N instructions instead of 10 N.
template <typename T, int N>
__device__ __forceinline__ T warp_sums(const T (&in)[N], int lane, int& k) {
  constexpr int NP2 = N <= 1 ? 1 : N <= 2 ? 2 : N <= 4 ? 4 : N <= 8 ? 8 : 16;
  static_assert(N <= 16, "at most 16 values");
  T v[NP2];
#pragma unroll
  for (int j = 0; j < NP2; ++j) v[j] = j < N ? in[j] : T(0);
  k = 0;
  int off = 16;
#pragma unroll
  for (int n = NP2; n > 1; n >>= 1, off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int j = 0; j < n / 2; ++j) {
      const T send = upper ? v[j] : v[j + n / 2];
      const T keep = upper ? v[j + n / 2] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    if (upper) k += n / 2;
  }
  for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
  if ((lane & (32 / NP2 - 1)) != 0 || k >= N) k = N;
  return v[0];
}

// Dynamic shared memory: [NM][C] message gradient of the target | G rows | dY partial sums.
template <typename T, typename TP, bool ENV, bool RT>
__device__ __forceinline__ void tp_bwd_row(const TPArgs<T>& a, int i, unsigned char* smem_raw, T* red_u, T* red_r, RtEdge<T>* rts,
                                           int* esrc) {
  const int c = threadIdx.x, C = a.C;
  const int nwarp = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  T* gMs = reinterpret_cast<T*>(smem_raw);          // [NM][C]
  T* Gs = gMs + TP::NM * C;                          // [kEdgeBatch][NG]
  T* red = Gs + kEdgeBatch * TP::NG;                 // [kEdgeBatch][8 warps][D]
  const int rt_first = blockDim.x > 32 ? 32 : 0;  // the second warp (when there is one) prepares the interpolation
  const int beg = a.rowptr[i], end = a.rowptr[i + 1];
  const T* gMi = a.gM + (long long)i * TP::NM * C;
  if (beg < end)
    for (int k = 0; k < TP::NM; ++k) gMs[k * C + c] = gMi[k * C + c];  // each thread reads and writes only its own column
  for (int e0 = beg; e0 < end; e0 += kEdgeBatch) {
    const int nb = min(kEdgeBatch, end - e0);
    __syncthreads();
    if (threadIdx.x < nb) esrc[threadIdx.x] = a.e_src[e0 + threadIdx.x];
    if (RT && (int)threadIdx.x >= rt_first && (int)threadIdx.x < rt_first + nb)
      rt_prepare<T, true>(a, a.dlen[e0 + threadIdx.x - rt_first], rts[threadIdx.x - rt_first]);
    build_G_rows<T, TP>(a.Y, e0, nb, 0, TP::NPART, Gs);
    __syncthreads();
    for (int e = 0; e < nb; ++e) {
      const long long s = esrc[e];
      T xv[TP::NX], dYp[TP::D], dx[TP::NX];
#pragma unroll
      for (int k = 0; k < TP::NX; ++k) { xv[k] = a.x[(s * TP::NX + k) * C + c]; dx[k] = T(0); }
#pragma unroll
      for (int k = 0; k < TP::D; ++k) dYp[k] = T(0);
      T u = T(1);
      if constexpr (ENV) u = a.env[e0 + e];
      T du_part = T(0);  // dE/d(envelope) of this channel: sum_p dE/dW_p W_p
      T dr_part = T(0);  // dE/d(length) through the tabulated weights: sum_p dE/dW_p dW_p/dd
      if constexpr (RT) {
        RtBwdWeights<T, TP, ENV> wf;
        wf.row = a.rtab + ((long long)rts[e].k * TP::NP * C + c) * 4;
        wf.stride = (long long)C * 4;
        wf.b0 = rts[e].b[0]; wf.b1 = rts[e].b[1]; wf.b2 = rts[e].b[2]; wf.b3 = rts[e].b[3];
        wf.d0 = rts[e].d[0]; wf.d1 = rts[e].d[1]; wf.d2 = rts[e].d[2]; wf.d3 = rts[e].d[3];
        wf.u = u;
        wf.start();
        TP::template bwd_w<T>(xv, gMs + c, C, Gs + e * TP::NG, wf, dYp, dx);
        dr_part = wf.dr;
        du_part = wf.du;
      } else {
        ArrayBwdWeights<T, TP, ENV> wf;
        const long long wbase = (long long)(e0 + e - a.e_base) * TP::NP * C + c;
        wf.W = a.W + wbase;
        wf.dW = a.dW + wbase;
        wf.C = C;
        wf.u = u;
        wf.start();
        TP::template bwd_w<T>(xv, gMs + c, C, Gs + e * TP::NG, wf, dYp, dx);
        du_part = wf.du;
      }
      if (a.dxe) {
        T* out = a.dxe + (long long)(e0 + e - a.e_base) * TP::NX * C;
#pragma unroll
        for (int k = 0; k < TP::NX; ++k) out[k * C + c] = dx[k];
      }
      {  // reduce dY over the channels of this warp
        int k;
        const T v = warp_sums<T, TP::D>(dYp, lane, k);
        if (k < TP::D) red[(e * 8 + warp) * TP::D + k] = v;
      }
      if constexpr (ENV) {  // the same reduction for the envelope gradient
        T v = du_part;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red_u[e * 8 + warp] = v;
      }
      if constexpr (RT) {  // and for the edge-length gradient through the tabulated weights
        T v = dr_part;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) red_r[e * 8 + warp] = v;
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
    if (RT && (int)threadIdx.x >= rt_first && (int)threadIdx.x < rt_first + nb) {
      const int e = threadIdx.x - rt_first;
      T v = T(0);
      for (int w = 0; w < nwarp; ++w) v += red_r[e * 8 + w];
      T* dst = a.ddlen + (e0 + e);
      *dst = a.accumulate_ddlen ? (*dst + v) : v;
    }
  }
}
template <typename T, typename TP, bool ENV, bool RT, bool LIST>
// register cap: rank 3 needs 168 to stay (nearly) free of spills; up to rank 2 fits 128, which lets two more blocks share an SM
__global__ void __maxnreg__(TP::L <= 2 ? 128 : 168) tp_bwd_kernel(const TPArgs<T> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ T red_u[kEdgeBatch * 8];                // envelope-gradient partial sums
  __shared__ T red_r[RT ? kEdgeBatch * 8 : 1];       // edge-length-gradient partial sums (tabulated weights)
  __shared__ RtEdge<T> rts[RT ? kEdgeBatch : 1];
  __shared__ int esrc[kEdgeBatch];
  if constexpr (LIST) {
    for (int it = blockIdx.x * kListRows; it < (blockIdx.x + 1) * kListRows; ++it) {
      const int i = tp_row(a, it);
      if (i < 0) break;
      tp_bwd_row<T, TP, ENV, RT>(a, i, smem_raw, red_u, red_r, rts, esrc);
    }
  } else {
    tp_bwd_row<T, TP, ENV, RT>(a, blockIdx.x, smem_raw, red_u, red_r, rts, esrc);
  }
}

// Backward pass of the first interaction (scalar source): the paths are (0, l, l), so the coupling is the identity,
// M[i, (l, m), c] = sum_e w[e, l, c] x[src_e, c] Y_e[l, m], and nothing flows back to the source features.  What costs
// here is not arithmetic but the sum over channels behind every dY_e[l, m].  Instead of D warp-shuffle reductions per
// edge the block works in two phases per batch of edges: (1) thread = channel writes z[e][l][c] = w x (and the
// per-channel terms of dE/d(length) and dE/d(envelope)) to shared memory and the weight gradient to global memory;
// (2) thread = (edge, component) walks over the channels, dY_e[l, m] = sum_c z[e][l][c] gM[i, (l, m), c], starting at a
// rotated channel so that the threads of a warp hit different banks.  Sums run in a fixed order: bit-reproducible.
template <typename T, typename TP, bool ENV, bool RT>
__global__ void tp_bwd_scalar_kernel(const TPArgs<T> a) {
  constexpr int D = TP::D, NP = TP::NP, EB = kEdgeBatch;
  static_assert(TP::NX == 1 && TP::NM == TP::D, "scalar source: one path per rank");
  extern __shared__ __align__(32) unsigned char smem_raw[];
  const int i = blockIdx.x, c = threadIdx.x, C = a.C;
  T* gMs = reinterpret_cast<T*>(smem_raw);  // [D][C]
  T* zs = gMs + D * C;                      // [EB][NP][C]
  T* rs = zs + EB * NP * C;                 // [EB][2][C]: per-channel dE/d(length) and dE/d(envelope) terms
  __shared__ T Ys[EB * D];
  __shared__ int esrc[EB];
  __shared__ T env_s[EB];
  __shared__ RtEdge<T> rts[RT ? EB : 1];
  const T* gMi = a.gM + (long long)i * D * C;
  for (int k = 0; k < D; ++k) gMs[k * C + c] = gMi[k * C + c];
  const int beg = a.rowptr[i], end = a.rowptr[i + 1];
  for (int e0 = beg; e0 < end; e0 += EB) {
    const int nb = min(EB, end - e0);
    __syncthreads();
    if (c < nb) {
      esrc[c] = a.e_src[e0 + c];
      if (ENV) env_s[c] = a.env[e0 + c];
      if (RT) rt_prepare<T, true>(a, a.dlen[e0 + c], rts[c]);
    }
    for (int idx = c; idx < nb * D; idx += blockDim.x) Ys[idx] = a.Y[(long long)e0 * D + idx];
    __syncthreads();
    // phase 1: thread = channel.  Four edges at a time: first every global load of the group (source feature, table
    // entries or weights) goes out, then the arithmetic runs, so the loads of four edges overlap instead of one.
    constexpr int SUB = 4;
    for (int eb = 0; eb < nb; eb += SUB) {
      T xs_[SUB], w_[SUB][NP], wd_[SUB][NP];
#pragma unroll
      for (int j = 0; j < SUB; ++j) {
        const int e = min(eb + j, nb - 1);  // lanes past the end repeat the last edge and are dropped below
        xs_[j] = a.x[(long long)esrc[e] * C + c];
        const long long wbase = (long long)(e0 + e - a.e_base) * NP * C;
#pragma unroll
        for (int l = 0; l < NP; ++l) {
          if constexpr (RT) {
            T v0, m0, v1, m1;
            rt_load<T>(a.rtab + ((long long)rts[e].k * NP * C + (long long)l * C + c) * 4, v0, m0, v1, m1);
            w_[j][l] = rts[e].b[0] * v0 + rts[e].b[1] * m0 + rts[e].b[2] * v1 + rts[e].b[3] * m1;
            wd_[j][l] = rts[e].d[0] * v0 + rts[e].d[1] * m0 + rts[e].d[2] * v1 + rts[e].d[3] * m1;
          } else {
            w_[j][l] = a.W[wbase + l * C + c];
            wd_[j][l] = T(0);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < SUB; ++j) {
        const int e = eb + j;
        if (e >= nb) break;
        const T xs = xs_[j];
        const T u = ENV ? env_s[e] : T(1);
        const long long wbase = (long long)(e0 + e - a.e_base) * NP * C;
        T dr_part = T(0), du_part = T(0);
        int lm = 0;
#pragma unroll
        for (int l = 0; l < NP; ++l) {
          T t = T(0);  // sum_m Y[l, m] gM[(l, m), c]
#pragma unroll
          for (int m = 0; m < 2 * l + 1; ++m, ++lm) t += Ys[e * D + lm] * gMs[lm * C + c];
          const T dw_eff = xs * t;  // gradient with respect to the (envelope-scaled) weight
          zs[(e * NP + l) * C + c] = u * w_[j][l] * xs;
          du_part += dw_eff * w_[j][l];
          if constexpr (RT) dr_part += u * dw_eff * wd_[j][l];
          else a.dW[wbase + l * C + c] = u * dw_eff;
        }
        rs[(e * 2 + 0) * C + c] = dr_part;
        rs[(e * 2 + 1) * C + c] = du_part;
      }
    }
    __syncthreads();
    // phase 2: thread = (edge, component) for dY, then one thread per edge for the two scalar sums
    for (int r = c; r < nb * D; r += blockDim.x) {
      const int e = r / D, lm = r - e * D;
      const int l = lm < 1 ? 0 : lm < 4 ? 1 : lm < 9 ? 2 : 3;
      // four channels per step (C is a multiple of 32), four partial sums, combined in a fixed order
      const RowVec<T, 4>* zr = reinterpret_cast<const RowVec<T, 4>*>(zs + (e * NP + l) * C);
      const RowVec<T, 4>* gr = reinterpret_cast<const RowVec<T, 4>*>(gMs + lm * C);
      const int C4 = C >> 2;
      int k = r % C4;  // rotated start: consecutive (edge, component) pairs of a warp start in different banks
      T p0 = T(0), p1 = T(0), p2 = T(0), p3 = T(0);
      for (int n = 0; n < C4; ++n) {
        const RowVec<T, 4> z = zr[k], g = gr[k];
        p0 += z.v[0] * g.v[0]; p1 += z.v[1] * g.v[1]; p2 += z.v[2] * g.v[2]; p3 += z.v[3] * g.v[3];
        k = k + 1 == C4 ? 0 : k + 1;
      }
      const T acc = (p0 + p1) + (p2 + p3);
      T* dst = a.dY + (long long)(e0 + e) * D + lm;
      *dst = a.accumulate_dY ? (*dst + acc) : acc;
    }
    const int first = blockDim.x > 32 ? 32 : 0;  // a second warp, when there is one, takes the scalar sums
    if ((RT || ENV) && c >= first && c < first + 2 * nb) {
      const int e = (c - first) >> 1, which = (c - first) & 1;
      if ((which == 0 && RT) || (which == 1 && ENV)) {
        const RowVec<T, 4>* rr = reinterpret_cast<const RowVec<T, 4>*>(rs + (e * 2 + which) * C);
        const int C4 = C >> 2;
        int k = (2 * e + which) % C4;
        T p0 = T(0), p1 = T(0), p2 = T(0), p3 = T(0);
        for (int n = 0; n < C4; ++n) {
          const RowVec<T, 4> x = rr[k];
          p0 += x.v[0]; p1 += x.v[1]; p2 += x.v[2]; p3 += x.v[3];
          k = k + 1 == C4 ? 0 : k + 1;
        }
        const T acc = (p0 + p1) + (p2 + p3);
        if (which == 0) {
          T* dst = a.ddlen + (e0 + e);
          *dst = a.accumulate_ddlen ? (*dst + acc) : acc;
        } else {
          T* dst = a.denv + (e0 + e);
          *dst = a.accumulate_denv ? (*dst + acc) : acc;
        }
      }
    }
  }
}

// V = T, or a 16-byte vector of T when the row length and the base addresses allow: every element is still summed over the
// edges in list order, so the result does not depend on the vector width.
template <typename T, int W>
__global__ void segment_sum_rows_kernel(const RowVec<T, W>* __restrict__ dxe, const int* __restrict__ rowptr, const int* __restrict__ perm,
                                        RowVec<T, W>* __restrict__ gx, int first, int row_len) {
  const int b = first + blockIdx.x;
  const int beg = rowptr[b], end = rowptr[b + 1];
  for (int k = threadIdx.x; k < row_len; k += blockDim.x) {
    RowVec<T, W> acc;
#pragma unroll
    for (int i = 0; i < W; ++i) acc.v[i] = T(0);
    for (int j = beg; j < end; ++j) {
      const RowVec<T, W> x = dxe[(long long)perm[j] * row_len + k];
#pragma unroll
      for (int i = 0; i < W; ++i) acc.v[i] += x.v[i];
    }
    gx[(long long)b * row_len + k] = acc;
  }
}
template <typename T>
cudaError_t launch_segment_sum_rows(const T* dxe, const int* rowptr_src, const int* perm_src, T* gx, int first_atom, int n_atoms,
                                    int row_len, cudaStream_t s) {
  if (n_atoms <= 0) return cudaSuccess;
  constexpr int W = 16 / sizeof(T);
  auto threads_for = [](int items) { const int t = (items + 31) / 32 * 32; return t < 32 ? 32 : (t > 256 ? 256 : t); };
  if (row_len % W == 0 && ((reinterpret_cast<uintptr_t>(dxe) | reinterpret_cast<uintptr_t>(gx)) & 15) == 0)
    segment_sum_rows_kernel<T, W><<<n_atoms, threads_for(row_len / W), 0, s>>>(reinterpret_cast<const RowVec<T, W>*>(dxe), rowptr_src, perm_src,
                                                            reinterpret_cast<RowVec<T, W>*>(gx), first_atom, row_len / W);
  else
    segment_sum_rows_kernel<T, 1><<<n_atoms, threads_for(row_len), 0, s>>>(reinterpret_cast<const RowVec<T, 1>*>(dxe), rowptr_src, perm_src,
                                                            reinterpret_cast<RowVec<T, 1>*>(gx), first_atom, row_len);
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

template <typename T, typename TP, bool ENV, bool RT>
cudaError_t launch_fwd_v(const TPArgs<T>& a, cudaStream_t s) {
  if (a.row_ids) {
    tp_fwd_kernel<T, TP, 0, ENV, RT, true><<<(a.n_seg + kListRows - 1) / kListRows, a.C, 0, s>>>(a);
    if (TP::NGRP > 1) tp_fwd_kernel<T, TP, 1, ENV, RT, true><<<(a.n_seg + kListRows - 1) / kListRows, a.C, 0, s>>>(a);
  } else {
    tp_fwd_kernel<T, TP, 0, ENV, RT, false><<<a.n_seg, a.C, 0, s>>>(a);
    if (TP::NGRP > 1) tp_fwd_kernel<T, TP, 1, ENV, RT, false><<<a.n_seg, a.C, 0, s>>>(a);
  }
  return cudaGetLastError();
}
template <typename T, typename TP>
cudaError_t launch_fwd_t(const TPArgs<T>& a, cudaStream_t s) {
  if (a.rtab) {
    if (!a.dlen || a.rt_K < 1) return cudaErrorInvalidValue;
    return a.env ? launch_fwd_v<T, TP, true, true>(a, s) : launch_fwd_v<T, TP, false, true>(a, s);
  }
  return a.env ? launch_fwd_v<T, TP, true, false>(a, s) : launch_fwd_v<T, TP, false, false>(a, s);
}
template <typename T, typename TP, bool RT>
cudaError_t launch_bwd_v(const TPArgs<T>& a, size_t smem, cudaStream_t s) {
  static size_t configured[64] = {};  // the attribute belongs to a device: one slot per device ordinal
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidValue;
  if (smem > 48 * 1024 && smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tp_bwd_kernel<T, TP, false, RT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tp_bwd_kernel<T, TP, true, RT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tp_bwd_kernel<T, TP, false, RT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tp_bwd_kernel<T, TP, true, RT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[dev] = smem;
  }
  if (a.row_ids) {
    if (a.env) tp_bwd_kernel<T, TP, true, RT, true><<<(a.n_seg + kListRows - 1) / kListRows, a.C, smem, s>>>(a);
    else tp_bwd_kernel<T, TP, false, RT, true><<<(a.n_seg + kListRows - 1) / kListRows, a.C, smem, s>>>(a);
  } else {
    if (a.env) tp_bwd_kernel<T, TP, true, RT, false><<<a.n_seg, a.C, smem, s>>>(a);
    else tp_bwd_kernel<T, TP, false, RT, false><<<a.n_seg, a.C, smem, s>>>(a);
  }
  return cudaGetLastError();
}
template <typename T, typename TP, bool ENV, bool RT>
cudaError_t launch_bwd_scalar(const TPArgs<T>& a, cudaStream_t s) {
  const size_t smem = sizeof(T) * ((size_t)TP::D * a.C + (size_t)kEdgeBatch * (TP::NP + 2) * a.C);
  static size_t configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return cudaErrorInvalidValue;
  if (smem > 48 * 1024 && smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tp_bwd_scalar_kernel<T, TP, ENV, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured[dev] = smem;
  }
  tp_bwd_scalar_kernel<T, TP, ENV, RT><<<a.n_seg, a.C, smem, s>>>(a);
  return cudaGetLastError();
}
template <typename T, typename TP>
cudaError_t launch_bwd_t(const TPArgs<T>& a, cudaStream_t s) {
  const size_t smem = sizeof(T) * ((size_t)TP::NM * a.C + kEdgeBatch * TP::NG + kEdgeBatch * 8 * TP::D);
  if (a.env && !a.denv) return cudaErrorInvalidValue;
  if constexpr (TP::NX == 1 && TP::NM == TP::D) {  // scalar source (first interaction): the two-phase kernel
    if (a.rtab && (!a.dlen || !a.ddlen || a.rt_K < 1)) return cudaErrorInvalidValue;
    if (a.rtab) return a.env ? launch_bwd_scalar<T, TP, true, true>(a, s) : launch_bwd_scalar<T, TP, false, true>(a, s);
    return a.env ? launch_bwd_scalar<T, TP, true, false>(a, s) : launch_bwd_scalar<T, TP, false, false>(a, s);
  }
  if (a.rtab) {
    if (!a.dlen || !a.ddlen || a.rt_K < 1) return cudaErrorInvalidValue;
    return launch_bwd_v<T, TP, true>(a, smem, s);
  }
  return launch_bwd_v<T, TP, false>(a, smem, s);
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
template cudaError_t launch_segment_sum_rows<float>(const float*, const int*, const int*, float*, int, int, int, cudaStream_t);
template cudaError_t launch_segment_sum_rows<double>(const double*, const int*, const int*, double*, int, int, int, cudaStream_t);
template cudaError_t launch_chunk_src_sum<float>(const float*, const int*, const int*, long long, long long, long long, float*, int, cudaStream_t);
template cudaError_t launch_chunk_src_sum<double>(const double*, const int*, const int*, long long, long long, long long, double*, int, cudaStream_t);

}  // namespace tace
