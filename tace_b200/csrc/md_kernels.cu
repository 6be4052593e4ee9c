// Molecular-dynamics support kernels for the domain-decomposed driver: velocity-Verlet updates,
// kinetic energy, edge vectors from fp64 positions, and the row gather / scatter-add used to pack and
// unpack halo messages.  All are single-pass streaming kernels (HBM-bound); state (positions,
// velocities) is fp64, forces arrive in the model's dtype.
//
// The reference has no integrator of its own: its MD runs go through LAMMPS (`fix nve`) or ASE; these
// entry points stand in for that host so a whole MD step stays on the device.
#include <cuda_runtime.h>
#include <cub/cub.cuh>
#include <cstdint>
#include <type_traits>

#include "../../include/tace_b200.h"

namespace tace {
namespace {

template <typename F>
__global__ void md_kick_drift_kernel(double* __restrict__ pos, double* __restrict__ vel, const F* __restrict__ forces,
                                     const double* __restrict__ inv_mass, long long n3, double kick, double dt) {
  const long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (k >= n3) return;
  double v = vel[k];
  if (forces) v += kick * (double)forces[k] * inv_mass[k / 3];
  vel[k] = v;
  if (pos) pos[k] += dt * v;
}

__global__ void md_kinetic_partial_kernel(const double* __restrict__ vel, const double* __restrict__ mass, long long n,
                                          double* __restrict__ partial) {
  __shared__ double red[256];
  double acc = 0.0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const double vx = vel[3 * i], vy = vel[3 * i + 1], vz = vel[3 * i + 2];
    acc += 0.5 * mass[i] * (vx * vx + vy * vy + vz * vz);
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}
__global__ void md_kinetic_final_kernel(const double* __restrict__ partial, int n_partial, double* out) {
  __shared__ double red[256];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n_partial; i += blockDim.x) acc += partial[i];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = red[0];
}

template <typename T>
__global__ void edge_vectors_kernel(const double* __restrict__ pos, const int64_t* __restrict__ edge_index, long long E,
                                    T* __restrict__ out) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= E) return;
  const long long s = edge_index[e], t = edge_index[E + e];
#pragma unroll
  for (int k = 0; k < 3; ++k) out[3 * e + k] = (T)(pos[3 * t + k] - pos[3 * s + k]);
}

// dst[r] = src[idx[r]]  (GATHER)   or   dst[idx[r]] += src[r]  (indices unique within one call)
template <typename V, bool GATHER>
__global__ void rows_kernel(const V* __restrict__ src, const int64_t* __restrict__ idx, long long n_rows, int row_len,
                            V* __restrict__ dst) {
  const long long total = n_rows * row_len;
  for (long long k = blockIdx.x * (long long)blockDim.x + threadIdx.x; k < total; k += (long long)gridDim.x * blockDim.x) {
    const long long r = k / row_len;
    const int c = (int)(k - r * row_len);
    if (GATHER) dst[k] = src[idx[r] * row_len + c];
    else {
      V* d = dst + idx[r] * row_len + c;
      *d = *d + src[k];
    }
  }
}

inline unsigned grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  const long long cap = 148LL * 16;
  return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace
}  // namespace tace

// ---- Langevin thermostat: exact Ornstein-Uhlenbeck update of the velocities ---------------------
// v <- c1 v + sqrt((1 - c1^2) kT / m) xi, xi standard normal.  The random numbers are a pure function of
// (seed, step, atom id, component), so a trajectory does not depend on how atoms are spread over ranks.
__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {  // splitmix64 finaliser
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__global__ void md_langevin_kernel(double* __restrict__ vel, const double* __restrict__ inv_mass, const long long* __restrict__ ids,
                                   long long n, double c1, double kt_scaled, unsigned long long seed, unsigned long long step) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long id = ids ? (unsigned long long)ids[i] : (unsigned long long)i;
  const unsigned long long key = mix64(mix64(seed) ^ mix64(step * 0xD1342543DE82EF95ull + 1) ^ (id * 0x2545F4914F6CDD1Dull));
  // four uniforms in (0, 1] -> two Box-Muller pairs (three of the four normals are used)
  double u[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) u[k] = ((double)(mix64(key + k) >> 11) + 1.0) * (1.0 / 9007199254740992.0);
  const double r0 = sqrt(-2.0 * log(u[0])), r1 = sqrt(-2.0 * log(u[2]));
  const double two_pi = 6.283185307179586;
  const double xi[3] = {r0 * cos(two_pi * u[1]), r0 * sin(two_pi * u[1]), r1 * cos(two_pi * u[3])};
  const double sigma = sqrt((1.0 - c1 * c1) * kt_scaled * inv_mass[i]);
#pragma unroll
  for (int k = 0; k < 3; ++k) vel[3 * i + k] = c1 * vel[3 * i + k] + sigma * xi[k];
}

using namespace tace;

extern "C" int tace_md_langevin(double* velocities, const double* inv_mass, const int64_t* ids, int64_t n_atoms, double c1,
                                double kt_scaled, uint64_t seed, uint64_t step, tace_stream_t stream) {
  if (!velocities || !inv_mass || n_atoms < 0 || !(c1 >= 0.0 && c1 <= 1.0) || kt_scaled < 0.0) return TACE_ERR_INVALID_ARGUMENT;
  if (n_atoms == 0) return TACE_OK;
  md_langevin_kernel<<<(unsigned)((n_atoms + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      velocities, inv_mass, reinterpret_cast<const long long*>(ids), n_atoms, c1, kt_scaled, seed, step);
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

extern "C" int tace_md_kick_drift(double* positions, double* velocities, const void* forces, int32_t force_dtype,
                                  const double* inv_mass, int64_t n_atoms, double kick, double dt, tace_stream_t stream) {
  if (!velocities || n_atoms < 0 || (forces && !inv_mass)) return TACE_ERR_INVALID_ARGUMENT;
  if (force_dtype != TACE_F32 && force_dtype != TACE_F64) return TACE_ERR_INVALID_ARGUMENT;
  if (n_atoms == 0) return TACE_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long n3 = 3 * n_atoms;
  const unsigned blocks = (unsigned)((n3 + 255) / 256);
  if (force_dtype == TACE_F32)
    md_kick_drift_kernel<float><<<blocks, 256, 0, s>>>(positions, velocities, static_cast<const float*>(forces), inv_mass, n3, kick, dt);
  else
    md_kick_drift_kernel<double><<<blocks, 256, 0, s>>>(positions, velocities, static_cast<const double*>(forces), inv_mass, n3, kick, dt);
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

extern "C" int tace_md_kinetic_energy(const double* velocities, const double* mass, int64_t n_atoms, double* scratch,
                                      double* out, tace_stream_t stream) {
  if (!velocities || !mass || !scratch || !out || n_atoms < 0) return TACE_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long blocks = (n_atoms + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 1024) blocks = 1024;
  md_kinetic_partial_kernel<<<(unsigned)blocks, 256, 0, s>>>(velocities, mass, n_atoms, scratch);
  md_kinetic_final_kernel<<<1, 256, 0, s>>>(scratch, (int)blocks, out);
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

extern "C" int tace_edge_vectors(const double* positions, const int64_t* edge_index, int64_t n_edges, void* out, int32_t dtype,
                                 tace_stream_t stream) {
  if (n_edges < 0 || (n_edges > 0 && (!positions || !edge_index || !out))) return TACE_ERR_INVALID_ARGUMENT;
  if (dtype != TACE_F32 && dtype != TACE_F64) return TACE_ERR_INVALID_ARGUMENT;
  if (n_edges == 0) return TACE_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((n_edges + 255) / 256);
  if (dtype == TACE_F32) edge_vectors_kernel<float><<<blocks, 256, 0, s>>>(positions, edge_index, n_edges, static_cast<float*>(out));
  else edge_vectors_kernel<double><<<blocks, 256, 0, s>>>(positions, edge_index, n_edges, static_cast<double*>(out));
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

// keep[e] = 1 where |r_target - r_source|^2 < cutoff^2, evaluated in fp64 with the neighbour-list kernel's own
// operation order (separately rounded products and sums), so a filtered skin list holds exactly the edges a fresh
// list with this cutoff would hold.
__global__ void edges_within_kernel(const double* __restrict__ pos, const long long* __restrict__ edge_index, long long n_edges,
                                    double cutoff, unsigned char* __restrict__ keep) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const long long s = edge_index[e], t = edge_index[n_edges + e];
  const double dx = __dadd_rn(pos[3 * t], -pos[3 * s]);
  const double dy = __dadd_rn(pos[3 * t + 1], -pos[3 * s + 1]);
  const double dz = __dadd_rn(pos[3 * t + 2], -pos[3 * s + 2]);
  const double dsq = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
  keep[e] = dsq < __dmul_rn(cutoff, cutoff) ? 1 : 0;
}

extern "C" int tace_edges_within(const double* positions, const int64_t* edge_index, int64_t n_edges, double cutoff,
                                 uint8_t* keep, tace_stream_t stream) {
  if (n_edges < 0 || !(cutoff > 0.0) || (n_edges > 0 && (!positions || !edge_index || !keep))) return TACE_ERR_INVALID_ARGUMENT;
  if (n_edges == 0) return TACE_OK;
  edges_within_kernel<<<(unsigned)((n_edges + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      positions, reinterpret_cast<const long long*>(edge_index), n_edges, cutoff, keep);
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

namespace tace {
// (a named namespace: the type is a template argument of a CUB kernel)
struct KeepToInt {
  __host__ __device__ int operator()(unsigned char k) const { return k ? 1 : 0; }
};
using KeepIterator = cub::TransformInputIterator<int, KeepToInt, const unsigned char*>;
namespace {
__global__ void edges_total_kernel(const unsigned char* __restrict__ keep, const int* __restrict__ position, long long n_edges,
                                   long long* total) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *total = (long long)position[n_edges - 1] + (keep[n_edges - 1] ? 1 : 0);
}
// the kept edges of a list, in list order, with their vectors r_target - r_source (fp64 difference, rounded once)
template <typename T>
__global__ void edges_compact_kernel(const double* __restrict__ pos, const long long* __restrict__ edge_index, long long n_edges,
                                     const unsigned char* __restrict__ keep, const int* __restrict__ position, long long n_kept,
                                     long long* __restrict__ out_index, T* __restrict__ out_vec) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= n_edges || !keep[e]) return;
  const long long k = position[e];
  if (k >= n_kept) return;
  const long long s = edge_index[e], t = edge_index[n_edges + e];
  out_index[k] = s;
  out_index[n_kept + k] = t;
#pragma unroll
  for (int d = 0; d < 3; ++d) out_vec[3 * k + d] = (T)(pos[3 * t + d] - pos[3 * s + d]);
}
}  // namespace
}  // namespace tace

extern "C" int tace_edges_scan_workspace_bytes(int64_t n_edges, size_t* bytes) {
  if (!bytes || n_edges < 0 || n_edges >= (1LL << 31)) return TACE_ERR_INVALID_ARGUMENT;
  size_t temp = 0;
  KeepIterator in(nullptr, tace::KeepToInt());
  if (cub::DeviceScan::ExclusiveSum(nullptr, temp, in, static_cast<int*>(nullptr), (int)n_edges) != cudaSuccess) return TACE_ERR_CUDA;
  *bytes = temp + 256;
  return TACE_OK;
}

extern "C" int tace_edges_scan(const uint8_t* keep, int64_t n_edges, int32_t* position, int64_t* total, void* workspace,
                               size_t workspace_bytes, tace_stream_t stream) {
  if (n_edges < 0 || n_edges >= (1LL << 31) || !total || (n_edges > 0 && (!keep || !position || !workspace))) return TACE_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n_edges == 0) return cudaMemsetAsync(total, 0, sizeof(int64_t), s) == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
  size_t need = 0;
  KeepIterator in(keep, tace::KeepToInt());
  if (cub::DeviceScan::ExclusiveSum(nullptr, need, in, position, (int)n_edges, s) != cudaSuccess) return TACE_ERR_CUDA;
  if (need > workspace_bytes) return TACE_ERR_CAPACITY;
  if (cub::DeviceScan::ExclusiveSum(workspace, need, in, position, (int)n_edges, s) != cudaSuccess) return TACE_ERR_CUDA;
  edges_total_kernel<<<1, 32, 0, s>>>(keep, position, n_edges, reinterpret_cast<long long*>(total));
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

extern "C" int tace_edges_compact(const double* positions, const int64_t* edge_index, int64_t n_edges, const uint8_t* keep,
                                  const int32_t* position, int64_t n_kept, int64_t* out_index, void* out_vec, int32_t dtype,
                                  tace_stream_t stream) {
  if (n_edges < 0 || n_kept < 0 || n_kept > n_edges || (dtype != TACE_F32 && dtype != TACE_F64)) return TACE_ERR_INVALID_ARGUMENT;
  if (n_kept == 0) return TACE_OK;
  if (!positions || !edge_index || !keep || !position || !out_index || !out_vec) return TACE_ERR_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((n_edges + 255) / 256);
  const long long* ei = reinterpret_cast<const long long*>(edge_index);
  long long* oi = reinterpret_cast<long long*>(out_index);
  if (dtype == TACE_F32) edges_compact_kernel<float><<<blocks, 256, 0, s>>>(positions, ei, n_edges, keep, position, n_kept, oi, static_cast<float*>(out_vec));
  else edges_compact_kernel<double><<<blocks, 256, 0, s>>>(positions, ei, n_edges, keep, position, n_kept, oi, static_cast<double*>(out_vec));
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

namespace {
template <bool GATHER>
int rows_dispatch(const void* src, const int64_t* idx, int64_t n_rows, int32_t row_len, int32_t elem_bytes, void* dst,
                  tace_stream_t stream) {
  if (n_rows < 0 || row_len <= 0 || (n_rows > 0 && (!src || !idx || !dst))) return TACE_ERR_INVALID_ARGUMENT;
  if (elem_bytes != 4 && elem_bytes != 8) return TACE_ERR_INVALID_ARGUMENT;
  if (n_rows == 0) return TACE_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = grid_for(n_rows * (long long)row_len, 256);
  // a gather moves bit patterns (any 4- or 8-byte type); a scatter-add treats them as float / double
  using V4 = typename std::conditional<GATHER, uint32_t, float>::type;
  using V8 = typename std::conditional<GATHER, uint64_t, double>::type;
  if (elem_bytes == 4)
    rows_kernel<V4, GATHER><<<blocks, 256, 0, s>>>(static_cast<const V4*>(src), idx, n_rows, row_len, static_cast<V4*>(dst));
  else
    rows_kernel<V8, GATHER><<<blocks, 256, 0, s>>>(static_cast<const V8*>(src), idx, n_rows, row_len, static_cast<V8*>(dst));
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}
}  // namespace

extern "C" int tace_rows_gather(const void* src, const int64_t* index, int64_t n_rows, int32_t row_len, int32_t elem_bytes,
                                void* dst, tace_stream_t stream) {
  return rows_dispatch<true>(src, index, n_rows, row_len, elem_bytes, dst, stream);
}
extern "C" int tace_rows_scatter_add(const void* src, const int64_t* index, int64_t n_rows, int32_t row_len, int32_t elem_bytes,
                                     void* dst, tace_stream_t stream) {
  return rows_dispatch<false>(src, index, n_rows, row_len, elem_bytes, dst, stream);
}
