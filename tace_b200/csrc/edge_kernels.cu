// Per-edge kernels: geometry, angular and radial features, hidden layers of the radial MLP
// (forward), and the chain rule back to the edge vector (backward); force and virial sums.
//
// One thread per edge.  The radial-MLP weights (67 KB in fp32 per layer) are read straight
// from global memory: every thread of a warp reads the same address, so each load is one
// L1-resident broadcast.
#include "kernels.h"

namespace tace {

template <typename T>
__device__ __forceinline__ void edge_geometry(const EdgeArgs<T>& a, long long e, T (&v)[3], T& d0, T& d) {
  const int eo = a.e_orig[e];
  if (a.edge_vector) {
    v[0] = a.edge_vector[3LL * eo + 0];
    v[1] = a.edge_vector[3LL * eo + 1];
    v[2] = a.edge_vector[3LL * eo + 2];
  } else {
    const long long s = a.e_src[e], t = a.e_dst[e];
    const T* lat = a.lattice + 9LL * a.atom_graph[s];
    const T s0 = a.shifts[3LL * eo + 0], s1 = a.shifts[3LL * eo + 1], s2 = a.shifts[3LL * eo + 2];
#pragma unroll
    for (int k = 0; k < 3; ++k)
      v[k] = (a.positions[3 * t + k] - a.positions[3 * s + k]) + (s0 * lat[k] + s1 * lat[3 + k] + s2 * lat[6 + k]);
  }
  d0 = sqrt(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
  d = d0 + T(1e-9);  // tace/models/adapter.py:347
}

template <typename T, int L>
__global__ void __launch_bounds__(128) edge_fwd_kernel(const EdgeArgs<T> a) {
  constexpr int D = (L + 1) * (L + 1);
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  T v[3], d0, d;
  edge_geometry(a, e, v, d0, d);
  a.vec[3 * e + 0] = v[0]; a.vec[3 * e + 1] = v[1]; a.vec[3 * e + 2] = v[2];
  const T inv = T(1) / d;
  T Y[D];
  sh_eval<T, L>(v[0] * inv, v[1] * inv, v[2] * inv, Y);
#pragma unroll
  for (int k = 0; k < D; ++k) a.Y[e * D + k] = Y[k];
  a.dlen[e] = d;
  if (a.env) {
    T u, du;
    envelope_eval<T>(d, a.rp, u, du);
    a.env[e] = u;
  }
}

// First layer of every radial MLP (8 -> 64, no activation yet): z1 = b(d) @ A0.  One thread per edge; the
// [edge][64] rows are transposed through shared memory so the block writes one contiguous chunk
// instead of 32 scattered 16-byte pieces per warp store.  The 64 -> 64 layers run as GEMMs.
template <typename T>
__global__ void __launch_bounds__(128) edge_mlp_in_kernel(const EdgeArgs<T> a) {
  __shared__ T tile[64][kHidden + 1];
  const long long e0 = blockIdx.x * (long long)blockDim.x;
  const long long e = e0 + threadIdx.x;
  const bool live = e < a.E;
  T b[kNumBessel];
  if (live) radial_eval<T>(a.dlen[e], a.rp, b, nullptr);
  for (int t = 0; t < a.n_layers; ++t) {
    T z[kHidden];
    if (live) {
#pragma unroll
      for (int j = 0; j < kHidden; ++j) z[j] = a.mlp[t].b0 ? a.mlp[t].b0[j] : T(0);
      if (a.mlp[t].tbl_dst) {  // species rows of the element-dependent edge update
        const T* rd = a.mlp[t].tbl_dst + (long long)a.species[a.e_dst[e]] * kHidden;
        const T* rs = a.mlp[t].tbl_src + (long long)a.species[a.e_src[e]] * kHidden;
#pragma unroll
        for (int j = 0; j < kHidden; ++j) z[j] += rd[j] + rs[j];
      }
#pragma unroll
      for (int k = 0; k < kNumBessel; ++k)
#pragma unroll
        for (int j4 = 0; j4 < kHidden / 4; ++j4) {
          T a0, a1, a2, a3;
          ld4(a.mlp[t].A0 + k * kHidden + 4 * j4, a0, a1, a2, a3);
          z[4 * j4] += b[k] * a0; z[4 * j4 + 1] += b[k] * a1; z[4 * j4 + 2] += b[k] * a2; z[4 * j4 + 3] += b[k] * a3;
        }
    }
    for (int half = 0; half < 2; ++half) {  // 64 rows at a time through the shared tile
      if (live && (threadIdx.x >> 6) == half) {
#pragma unroll
        for (int j = 0; j < kHidden; ++j) tile[threadIdx.x & 63][j] = z[j];
      }
      __syncthreads();
      const long long r0 = e0 + 64 * half;
      const long long n_live = a.E - r0 < 64 ? a.E - r0 : 64;
      T* out = a.Z1[t] + r0 * kHidden;
      T* act = a.H1[t] + r0 * kHidden;
      for (long long idx = threadIdx.x; idx < n_live * kHidden; idx += blockDim.x) {
        const T z1 = tile[idx / kHidden][idx % kHidden];
        out[idx] = z1;
        act[idx] = silu_(z1);
      }
      __syncthreads();
    }
  }
}

// dE/dd: back through the first MLP layer and the radial basis.  dH1 = dE/d(silu(z1)).
template <typename T>
__global__ void __launch_bounds__(128) edge_mlp_out_kernel(const EdgeArgs<T> a) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  T b[kNumBessel], dbdd[kNumBessel];
  radial_eval<T>(a.dlen[e], a.rp, b, dbdd);
  T dd = T(0);
  for (int t = 0; t < a.n_layers; ++t) {
    const T* g = a.dH1[t] + e * kHidden;
    const T* z = a.Z1[t] + e * kHidden;
    T db[kNumBessel];
#pragma unroll
    for (int k = 0; k < kNumBessel; ++k) db[k] = T(0);
#pragma unroll
    for (int j4 = 0; j4 < kHidden / 4; ++j4) {
      T g0, g1, g2, g3, z0, z1, z2, z3;
      ld4(g + 4 * j4, g0, g1, g2, g3);
      ld4(z + 4 * j4, z0, z1, z2, z3);
      // dH1 already holds dE/dz1 when the layer has a LayerNorm (ln_silu_bwd ran over it)
      const T d0 = a.dz1_given ? g0 : g0 * silu_grad_(z0), d1 = a.dz1_given ? g1 : g1 * silu_grad_(z1),
              d2 = a.dz1_given ? g2 : g2 * silu_grad_(z2), d3 = a.dz1_given ? g3 : g3 * silu_grad_(z3);
#pragma unroll
      for (int k = 0; k < kNumBessel; ++k) {
        T a0, a1, a2, a3;
        ld4(a.mlp[t].A0 + k * kHidden + 4 * j4, a0, a1, a2, a3);
        db[k] += d0 * a0 + d1 * a1 + d2 * a2 + d3 * a3;
      }
    }
#pragma unroll
    for (int k = 0; k < kNumBessel; ++k) dd += db[k] * dbdd[k];
  }
  if (a.denv && a.add_denv) {  // W = envelope * MLP: the envelope's own derivative
    T u, du;
    envelope_eval<T>(a.dlen[e], a.rp, u, du);
    dd += a.denv[e] * du;
  }
  a.ddlen[e] = a.accumulate_ddlen ? a.ddlen[e] + dd : dd;
}

template <typename T>
__global__ void silu_kernel(const T* __restrict__ in, T* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) out[i] = silu_(in[i]);
}
template <typename T>
__global__ void silu_grad_mul_kernel(T* __restrict__ g, const T* __restrict__ z, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) g[i] *= silu_grad_(z[i]);
}
// LayerNorm over the 64 features of a row (torch.nn.LayerNorm: biased variance, eps 1e-5, affine) followed by SiLU, as the
// reference's radial MLP has it between a hidden linear and its activation when the edge features carry species
// embeddings (tace/models/mlp.py:172-176, tace/models/_e3nn/base.py:183-185).  One warp per row, two features per lane.
constexpr double kLnEps = 1e-5;
template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T>
__global__ void __launch_bounds__(256) ln_silu_fwd_kernel(const T* __restrict__ z, const T* __restrict__ gamma,
                                                          const T* __restrict__ beta, T* __restrict__ h, long long rows) {
  const int lane = threadIdx.x & 31;
  const long long r = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T z0 = z[r * kHidden + lane], z1 = z[r * kHidden + 32 + lane];
  const T mean = warp_sum(z0 + z1) * T(1.0 / kHidden);
  const T c0 = z0 - mean, c1 = z1 - mean;
  const T rstd = T(1) / sqrt(warp_sum(c0 * c0 + c1 * c1) * T(1.0 / kHidden) + T(kLnEps));
  h[r * kHidden + lane] = silu_(c0 * rstd * gamma[lane] + beta[lane]);
  h[r * kHidden + 32 + lane] = silu_(c1 * rstd * gamma[32 + lane] + beta[32 + lane]);
}
// g <- dE/dz given g = dE/d(silu(LN(z))); the row statistics are recomputed from z
template <typename T>
__global__ void __launch_bounds__(256) ln_silu_bwd_kernel(T* __restrict__ g, const T* __restrict__ z, const T* __restrict__ gamma,
                                                          const T* __restrict__ beta, long long rows) {
  const int lane = threadIdx.x & 31;
  const long long r = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const T z0 = z[r * kHidden + lane], z1 = z[r * kHidden + 32 + lane];
  const T mean = warp_sum(z0 + z1) * T(1.0 / kHidden);
  const T c0 = z0 - mean, c1 = z1 - mean;
  const T rstd = T(1) / sqrt(warp_sum(c0 * c0 + c1 * c1) * T(1.0 / kHidden) + T(kLnEps));
  const T n0 = c0 * rstd, n1 = c1 * rstd;  // normalised features
  const T d0 = g[r * kHidden + lane] * silu_grad_(n0 * gamma[lane] + beta[lane]) * gamma[lane];
  const T d1 = g[r * kHidden + 32 + lane] * silu_grad_(n1 * gamma[32 + lane] + beta[32 + lane]) * gamma[32 + lane];
  const T m1 = warp_sum(d0 + d1) * T(1.0 / kHidden);
  const T m2 = warp_sum(d0 * n0 + d1 * n1) * T(1.0 / kHidden);
  g[r * kHidden + lane] = rstd * (d0 - m1 - n0 * m2);
  g[r * kHidden + 32 + lane] = rstd * (d1 - m1 - n1 * m2);
}
template <typename T>
cudaError_t launch_ln_silu_fwd(const T* z, const T* gamma, const T* beta, T* h, long long rows, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  ln_silu_fwd_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(z, gamma, beta, h, rows);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_ln_silu_bwd(T* g, const T* z, const T* gamma, const T* beta, long long rows, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  ln_silu_bwd_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(g, z, gamma, beta, rows);
  return cudaGetLastError();
}
// ---- learned edge density (scatter_norm = density) ----------------------------------------------
template <typename T>
__device__ __forceinline__ void density_edge(const DensityArgs<T>& a, T d, T& rho, T& drho) {
  T b[kNumBessel], db[kNumBessel];
  radial_eval<T>(d, a.rp, b, db);
  T y = a.b1 ? a.b1[0] : T(0), dy = T(0);
  for (int j = 0; j < kHidden; ++j) {
    T z = a.b0 ? a.b0[j] : T(0), dz = T(0);
#pragma unroll
    for (int k = 0; k < kNumBessel; ++k) { z += b[k] * a.A0[k * kHidden + j]; dz += db[k] * a.A0[k * kHidden + j]; }
    y += silu_(z) * a.w1[j];
    dy += silu_grad_(z) * dz * a.w1[j];
  }
  const T t = tanh(y * y);
  rho = t;
  drho = (T(1) - t * t) * T(2) * y * dy;
  if (a.use_env) {
    T u, du;
    envelope_eval<T>(d, a.rp, u, du);
    drho = drho * u + t * du;
    rho = t * u;
  }
}
template <typename T>
__global__ void density_fwd_kernel(const DensityArgs<T> a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.n) return;
  T acc = T(0);
  for (int e = a.rowptr_dst[i]; e < a.rowptr_dst[i + 1]; ++e) {
    T rho, drho;
    density_edge(a, a.dlen[e], rho, drho);
    acc += rho;
  }
  const T dens = acc * a.ab[1] + a.ab[0];
  a.inv_density[i] = dens == T(0) ? T(1e9) : T(1) / dens;
}
template <typename T>
__global__ void density_bwd_kernel(const DensityArgs<T> a) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  T rho, drho;
  density_edge(a, a.dlen[e], rho, drho);
  a.ddlen[e] += a.gdens[a.e_dst[e]] * a.ab[1] * drho;
}
template <typename T>
cudaError_t launch_density_fwd(const DensityArgs<T>& a, cudaStream_t s) {
  if (a.n <= 0) return cudaSuccess;
  density_fwd_kernel<T><<<(a.n + 63) / 64, 64, 0, s>>>(a);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_density_bwd(const DensityArgs<T>& a, cudaStream_t s) {
  if (a.E <= 0) return cudaSuccess;
  density_bwd_kernel<T><<<(unsigned)((a.E + 127) / 128), 128, 0, s>>>(a);
  return cudaGetLastError();
}

// ---- ZBL pair repulsion (tace/models/radial.py:788-874) ------------------------------------------
// energy of one directed edge (half of the pair energy) and its derivative with respect to the edge length
template <typename T>
__device__ __forceinline__ void zbl_pair(const ZblArgs<T>& a, int su, int sv, T d, T& v, T& dv) {
  const T zu = a.z[su], zv = a.z[sv];
  const T inv_a = (pow(zu, a.par[1]) + pow(zv, a.par[1])) / a.par[0];
  const T x = d * inv_a;
  const T c[4] = {T(0.1818), T(0.5099), T(0.2802), T(0.02817)};
  const T k[4] = {T(3.2), T(0.9423), T(0.4028), T(0.2016)};
  T phi = T(0), dphi = T(0);  // screening function and d phi / d d
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const T t = c[q] * exp(-k[q] * x);
    phi += t; dphi -= k[q] * inv_a * t;
  }
  RadialParams<T> rp;
  rp.rc = a.rcov[su] + a.rcov[sv]; rp.p = a.p;
  T u, du;
  envelope_eval<T>(d, rp, u, du);
  const T pref = T(0.5 * 14.3996) * zu * zv;
  const T coul = pref / d;
  v = coul * phi * u;
  dv = coul * ((dphi - phi / d) * u + phi * du);
}
template <typename T>
__global__ void zbl_fwd_kernel(const ZblArgs<T> a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.n) return;
  const int sv = a.species[i];
  T acc = T(0);
  for (int e = a.rowptr_dst[i]; e < a.rowptr_dst[i + 1]; ++e) {
    T v, dv;
    zbl_pair(a, a.species[a.e_src[e]], sv, a.dlen[e], v, dv);
    acc += v;
  }
  a.node[i] = acc;
}
template <typename T>
__global__ void zbl_bwd_kernel(const ZblArgs<T> a) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  const int i = a.e_dst[e];
  T v, dv;
  zbl_pair(a, a.species[a.e_src[e]], a.species[i], a.dlen[e], v, dv);
  a.ddlen[e] += (a.factor ? a.factor[i] : T(1)) * dv;
}
template <typename T>
cudaError_t launch_zbl_fwd(const ZblArgs<T>& a, cudaStream_t s) {
  if (a.n <= 0) return cudaSuccess;
  zbl_fwd_kernel<T><<<(a.n + 127) / 128, 128, 0, s>>>(a);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_zbl_bwd(const ZblArgs<T>& a, cudaStream_t s) {
  if (a.E <= 0) return cudaSuccess;
  zbl_bwd_kernel<T><<<(unsigned)((a.E + 255) / 256), 256, 0, s>>>(a);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_silu(const T* in, T* out, long long n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const long long blocks = (n + 255) / 256;
  silu_kernel<T><<<(unsigned)(blocks < 148 * 32 ? blocks : 148 * 32), 256, 0, s>>>(in, out, n);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_silu_grad_mul(T* g, const T* z, long long n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  const long long blocks = (n + 255) / 256;
  silu_grad_mul_kernel<T><<<(unsigned)(blocks < 148 * 32 ? blocks : 148 * 32), 256, 0, s>>>(g, z, n);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_edge_mlp_in(const EdgeArgs<T>& a, cudaStream_t s) {
  if (a.E <= 0) return cudaSuccess;
  edge_mlp_in_kernel<T><<<(unsigned)((a.E + 127) / 128), 128, 0, s>>>(a);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_edge_mlp_out(const EdgeArgs<T>& a, cudaStream_t s) {
  if (a.E <= 0) return cudaSuccess;
  edge_mlp_out_kernel<T><<<(unsigned)((a.E + 127) / 128), 128, 0, s>>>(a);
  return cudaGetLastError();
}

template <typename T, int L>
__global__ void __launch_bounds__(128) edge_bwd_kernel(const EdgeArgs<T> a) {
  constexpr int D = (L + 1) * (L + 1);
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= a.E) return;
  T v[3], d0, d;
  edge_geometry(a, e, v, d0, d);
  const T dd = a.ddlen[e];
  const T inv = T(1) / d;
  T dY[D], dn[3], g[3];
#pragma unroll
  for (int k = 0; k < D; ++k) dY[k] = a.dY[e * D + k];
  sh_grad<T, L>(v[0] * inv, v[1] * inv, v[2] * inv, dY, dn);
  edge_vector_grad<T>(v, d0, d, dd, dn, g);
  if (a.gvec_extra) { g[0] += a.gvec_extra[3 * e]; g[1] += a.gvec_extra[3 * e + 1]; g[2] += a.gvec_extra[3 * e + 2]; }
  a.g[3 * e + 0] = g[0]; a.g[3 * e + 1] = g[1]; a.g[3 * e + 2] = g[2];
  if (a.edge_forces) {
    const long long eo = a.e_orig[e];
    a.edge_forces[3 * eo + 0] = g[0]; a.edge_forces[3 * eo + 1] = g[1]; a.edge_forces[3 * eo + 2] = g[2];
  }
}

template <typename T>
cudaError_t launch_edge_fwd(const EdgeArgs<T>& a, cudaStream_t s) {
  if (a.E <= 0) return cudaSuccess;
  const unsigned grid = (unsigned)((a.E + 127) / 128);
  if (a.L == 1) edge_fwd_kernel<T, 1><<<grid, 128, 0, s>>>(a);
  else if (a.L == 2) edge_fwd_kernel<T, 2><<<grid, 128, 0, s>>>(a);
  else if (a.L == 3) edge_fwd_kernel<T, 3><<<grid, 128, 0, s>>>(a);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_edge_bwd(const EdgeArgs<T>& a, cudaStream_t s) {
  if (a.E <= 0) return cudaSuccess;
  const unsigned grid = (unsigned)((a.E + 127) / 128);
  if (a.L == 1) edge_bwd_kernel<T, 1><<<grid, 128, 0, s>>>(a);
  else if (a.L == 2) edge_bwd_kernel<T, 2><<<grid, 128, 0, s>>>(a);
  else if (a.L == 3) edge_bwd_kernel<T, 3><<<grid, 128, 0, s>>>(a);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ---- forces and virials ------------------------------------------------------------------------
template <typename T>
__global__ void forces_kernel(const ForceArgs<T> a) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.n_atoms) return;
  T f[3] = {T(0), T(0), T(0)};
  T w[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) w[k] = T(0);
  if (i < a.n_local) {
    for (int e = a.rowptr_dst[i]; e < a.rowptr_dst[i + 1]; ++e) {
      const T g0 = a.g[3LL * e], g1 = a.g[3LL * e + 1], g2 = a.g[3LL * e + 2];
      f[0] -= g0; f[1] -= g1; f[2] -= g2;
      if (a.atom_virial) {
        const T v0 = a.vec[3LL * e], v1 = a.vec[3LL * e + 1], v2 = a.vec[3LL * e + 2];
        w[0] += v0 * g0; w[1] += v0 * g1; w[2] += v0 * g2;
        w[3] += v1 * g0; w[4] += v1 * g1; w[5] += v1 * g2;
        w[6] += v2 * g0; w[7] += v2 * g1; w[8] += v2 * g2;
      }
    }
    if (a.atom_virial)
      for (int k = 0; k < 9; ++k) a.atom_virial[9LL * i + k] = w[k];
  }
  if (a.forces) {
    for (int k = a.rowptr_src[i]; k < a.rowptr_src[i + 1]; ++k) {
      const long long e = a.perm_src[k];
      f[0] += a.g[3 * e]; f[1] += a.g[3 * e + 1]; f[2] += a.g[3 * e + 2];
    }
    a.forces[3LL * i] = f[0]; a.forces[3LL * i + 1] = f[1]; a.forces[3LL * i + 2] = f[2];
  }
}
template <typename T>
cudaError_t launch_forces(const ForceArgs<T>& a, cudaStream_t s) {
  if (a.n_atoms <= 0) return cudaSuccess;
  forces_kernel<T><<<(a.n_atoms + 127) / 128, 128, 0, s>>>(a);
  return cudaGetLastError();
}

template <typename T>
__global__ void graph_virial_kernel(const T* __restrict__ atom_virial, const int* __restrict__ graph_ptr,
                                    const T* __restrict__ lattice, T* virials, T* stress) {
  __shared__ T red[9][128];
  const int g = blockIdx.x;
  T w[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) w[k] = T(0);
  for (int i = graph_ptr[g] + threadIdx.x; i < graph_ptr[g + 1]; i += blockDim.x)
#pragma unroll
    for (int k = 0; k < 9; ++k) w[k] += atom_virial[9LL * i + k];
#pragma unroll
  for (int k = 0; k < 9; ++k) red[k][threadIdx.x] = w[k];
  __syncthreads();
  for (int off = 64; off > 0; off >>= 1) {
    if (threadIdx.x < off)
#pragma unroll
      for (int k = 0; k < 9; ++k) red[k][threadIdx.x] += red[k][threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x < 9) {
    const int r = threadIdx.x / 3, c = threadIdx.x % 3;
    const T sym = T(0.5) * (red[3 * r + c][0] + red[3 * c + r][0]);  // dE/d(strain)
    if (virials) virials[9LL * g + threadIdx.x] = -sym;
    if (stress) {
      const T* m = lattice + 9LL * g;
      const T det = m[0] * (m[4] * m[8] - m[5] * m[7]) - m[1] * (m[3] * m[8] - m[5] * m[6]) + m[2] * (m[3] * m[7] - m[4] * m[6]);
      const T st = sym / fabs(det);
      stress[9LL * g + threadIdx.x] = (fabs(st) < T(1e10)) ? st : T(0);  // tace/models/adapter.py:114-115
    }
  }
}
template <typename T>
cudaError_t launch_graph_virial(const T* atom_virial, const int* graph_ptr, const T* lattice, T* virials, T* stress,
                                int n_graphs, cudaStream_t s) {
  if (n_graphs <= 0) return cudaSuccess;
  graph_virial_kernel<T><<<n_graphs, 128, 0, s>>>(atom_virial, graph_ptr, lattice, virials, stress);
  return cudaGetLastError();
}

#define INST(T)                                                                                      \
  template cudaError_t launch_edge_fwd<T>(const EdgeArgs<T>&, cudaStream_t);                         \
  template cudaError_t launch_edge_bwd<T>(const EdgeArgs<T>&, cudaStream_t);                         \
  template cudaError_t launch_edge_mlp_in<T>(const EdgeArgs<T>&, cudaStream_t);                      \
  template cudaError_t launch_edge_mlp_out<T>(const EdgeArgs<T>&, cudaStream_t);                     \
  template cudaError_t launch_silu<T>(const T*, T*, long long, cudaStream_t);                        \
  template cudaError_t launch_zbl_fwd<T>(const ZblArgs<T>&, cudaStream_t);                           \
  template cudaError_t launch_density_fwd<T>(const DensityArgs<T>&, cudaStream_t);                   \
  template cudaError_t launch_density_bwd<T>(const DensityArgs<T>&, cudaStream_t);                   \
  template cudaError_t launch_zbl_bwd<T>(const ZblArgs<T>&, cudaStream_t);                           \
  template cudaError_t launch_ln_silu_fwd<T>(const T*, const T*, const T*, T*, long long, cudaStream_t); \
  template cudaError_t launch_ln_silu_bwd<T>(T*, const T*, const T*, const T*, long long, cudaStream_t); \
  template cudaError_t launch_silu_grad_mul<T>(T*, const T*, long long, cudaStream_t);               \
  template cudaError_t launch_forces<T>(const ForceArgs<T>&, cudaStream_t);                          \
  template cudaError_t launch_graph_virial<T>(const T*, const int*, const T*, T*, T*, int, cudaStream_t);
INST(float)
INST(double)

}  // namespace tace
