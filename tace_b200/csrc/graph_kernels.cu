// Graph preparation: from the caller's edge_index (any order) to target-sorted and
// source-sorted CSR views, the atom -> graph map, and the species-sorted atom permutation used
// by the per-species linear layers.  Stable radix sorts (CUB) keep every ordering
// deterministic, which makes the segmented sums downstream bit-reproducible.
#include <cub/cub.cuh>
#include "kernels.h"

namespace tace {

namespace {

__global__ void iota_and_key_kernel(const int64_t* __restrict__ key_src, int* keys, int* vals, long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  keys[i] = (int)key_src[i];
  vals[i] = (int)i;
}
__global__ void iota_and_key32_kernel(const int* __restrict__ key_src, int* keys, int* vals, long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  keys[i] = key_src[i];
  vals[i] = (int)i;
}
__global__ void gather_src_kernel(const int64_t* __restrict__ src_row, const int* __restrict__ e_orig, int* e_src, long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  e_src[i] = (int)src_row[e_orig[i]];
}
// keys[i] = 1 if any edge into target i comes from a ghost atom (index >= n_local), else 0; vals[i] = i
__global__ void ghost_row_key_kernel(const int* __restrict__ rowptr, const int* __restrict__ e_src, int n_local, int* keys, int* vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_local) return;
  int flag = 0;
  for (int e = rowptr[i]; e < rowptr[i + 1]; ++e) flag |= (e_src[e] >= n_local) ? 1 : 0;
  keys[i] = flag;
  vals[i] = i;
}
// rowptr[i] = number of sorted keys < i, i = 0..n_rows
__global__ void lower_bound_kernel(const int* __restrict__ sorted_keys, long long n_keys, int* rowptr, int n_rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n_rows) return;
  long long lo = 0, hi = n_keys;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (sorted_keys[mid] < i) lo = mid + 1; else hi = mid;
  }
  rowptr[i] = (int)lo;
}
__global__ void atom_graph_kernel(const int* __restrict__ graph_ptr, int n_graphs, int* atom_graph, int n_atoms) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_atoms) return;
  int lo = 0, hi = n_graphs;  // largest g with graph_ptr[g] <= i
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (graph_ptr[mid] <= i) lo = mid; else hi = mid;
  }
  atom_graph[i] = lo;
}
// tile_ptr: 64-row tiles of the CUDA-core GEMM; tc_tile_ptr: (128 / q)-atom tiles of the tensor-core GEMM
__global__ void tile_ptr_kernel(const int* __restrict__ species_ptr, int n_el, int* tile_ptr, int* tc_tile_ptr) {
  const int qi = threadIdx.x & 3;  // q = 2*qi + 1
  const bool tc = threadIdx.x >= 4;
  if (threadIdx.x >= 8) return;
  const int q = 2 * qi + 1;
  int* tp = (tc ? tc_tile_ptr : tile_ptr) + qi * (n_el + 1);
  const int R = 128 / q;
  int acc = 0;
  for (int g = 0; g < n_el; ++g) {
    tp[g] = acc;
    const int cnt = species_ptr[g + 1] - species_ptr[g];
    acc += tc ? (cnt + R - 1) / R : (cnt * q + 63) / 64;
  }
  tp[n_el] = acc;
}

__global__ void chunk_bounds_kernel(const int* __restrict__ rowptr, int n_local, long long target, int n_chunks, int* atom_ptr,
                                    int* edge_ptr) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c > n_chunks) return;
  int a = n_local;
  if (c < n_chunks) {  // first atom whose edge offset is >= c * target
    const long long want = c * target;
    int lo = 0, hi = n_local;
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (rowptr[mid] < want) lo = mid + 1; else hi = mid; }
    a = lo;
  }
  atom_ptr[c] = a;
  edge_ptr[c] = rowptr[a];
}
__global__ void chunk_key_kernel(const int* __restrict__ e_src, long long E, int n_atoms, const int* __restrict__ edge_ptr,
                                 int n_chunks, int* keys, int* vals) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (e >= E) return;
  int lo = 0, hi = n_chunks;  // largest c with edge_ptr[c] <= e
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (edge_ptr[mid] <= e) lo = mid; else hi = mid; }
  keys[e] = lo * n_atoms + e_src[e];
  vals[e] = (int)e;
}

inline size_t align_up(size_t x) { return (x + 255) & ~size_t(255); }

size_t cub_sort_bytes(long long n) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const int*)nullptr, (int*)nullptr, (const int*)nullptr, (int*)nullptr,
                                  (int)n);
  return bytes;
}

}  // namespace

size_t graph_prep_temp_bytes(long long E, int n_atoms) {
  const long long n = E > n_atoms ? E : n_atoms;
  return 3 * align_up(sizeof(int) * (size_t)n) + align_up(cub_sort_bytes(n)) + 256;
}

cudaError_t launch_graph_prep(const GraphPrepArgs& a, cudaStream_t s) {
  const long long n = a.E > a.n_atoms ? a.E : a.n_atoms;
  unsigned char* p = static_cast<unsigned char*>(a.temp);
  int* keys_in = reinterpret_cast<int*>(p); p += align_up(sizeof(int) * (size_t)n);
  int* vals_in = reinterpret_cast<int*>(p); p += align_up(sizeof(int) * (size_t)n);
  int* keys_out = reinterpret_cast<int*>(p); p += align_up(sizeof(int) * (size_t)n);
  void* cub_temp = p;
  size_t cub_bytes = cub_sort_bytes(n);
  if ((size_t)(p - static_cast<unsigned char*>(a.temp)) + cub_bytes > a.temp_bytes) return cudaErrorInvalidValue;
  int bits = 1;
  while ((1LL << bits) < (long long)a.n_atoms + 1 && bits < 31) ++bits;
  cudaError_t err;

  if (a.n_atoms > 0) atom_graph_kernel<<<(a.n_atoms + 255) / 256, 256, 0, s>>>(a.graph_ptr, a.n_graphs, a.atom_graph, a.n_atoms);

  if (a.E > 0) {
    const unsigned eb = (unsigned)((a.E + 255) / 256);
    // target-sorted view
    iota_and_key_kernel<<<eb, 256, 0, s>>>(a.edge_index + a.E, keys_in, vals_in, a.E);
    err = cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, keys_in, a.e_dst, vals_in, a.e_orig, (int)a.E, 0, bits, s);
    if (err != cudaSuccess) return err;
    gather_src_kernel<<<eb, 256, 0, s>>>(a.edge_index, a.e_orig, a.e_src, a.E);
    // source-sorted view over the target-sorted numbering
    iota_and_key32_kernel<<<eb, 256, 0, s>>>(a.e_src, keys_in, vals_in, a.E);
    err = cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, keys_in, keys_out, vals_in, a.perm_src, (int)a.E, 0, bits, s);
    if (err != cudaSuccess) return err;
  }
  lower_bound_kernel<<<(a.n_local + 256) / 256, 256, 0, s>>>(a.e_dst, a.E, a.rowptr_dst, a.n_local);
  lower_bound_kernel<<<(a.n_atoms + 256) / 256, 256, 0, s>>>(keys_out, a.E, a.rowptr_src, a.n_atoms);

  if (a.split_rows && a.n_local > 0) {  // stable one-bit sort: targets without a ghost source first
    ghost_row_key_kernel<<<(a.n_local + 255) / 256, 256, 0, s>>>(a.rowptr_dst, a.e_src, a.n_local, keys_in, vals_in);
    err = cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, keys_in, keys_out, vals_in, a.row_ids, a.n_local, 0, 1, s);
    if (err != cudaSuccess) return err;
    lower_bound_kernel<<<1, 32, 0, s>>>(keys_out, a.n_local, a.row_split, 1);
  }

  // species-sorted permutation of the local atoms (none on a rank that owns no atom: the row pointers below are all 0)
  int sbits = 1;
  while ((1 << sbits) < a.n_elements + 1 && sbits < 31) ++sbits;
  if (a.n_local > 0) {
    iota_and_key32_kernel<<<(a.n_local + 255) / 256, 256, 0, s>>>(a.species, keys_in, vals_in, a.n_local);
    err = cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, keys_in, keys_out, vals_in, a.species_perm, a.n_local, 0, sbits, s);
    if (err != cudaSuccess) return err;
  }
  lower_bound_kernel<<<(a.n_elements + 256) / 256, 256, 0, s>>>(keys_out, a.n_local, a.species_ptr, a.n_elements);
  tile_ptr_kernel<<<1, 32, 0, s>>>(a.species_ptr, a.n_elements, a.tile_ptr, a.tc_tile_ptr);
  return cudaGetLastError();
}

cudaError_t launch_chunk_bounds(const int* rowptr_dst, int n_local, long long target_edges, int n_chunks, int* atom_ptr,
                                int* edge_ptr, cudaStream_t s) {
  chunk_bounds_kernel<<<(n_chunks + 128) / 128, 128, 0, s>>>(rowptr_dst, n_local, target_edges, n_chunks, atom_ptr, edge_ptr);
  return cudaGetLastError();
}

cudaError_t launch_chunk_src_sort(const int* e_src, long long E, int n_atoms, const int* edge_ptr, int n_chunks, int* keys,
                                  int* perm, void* temp, size_t temp_bytes, cudaStream_t s) {
  if (E <= 0) return cudaSuccess;
  if ((long long)n_chunks * n_atoms >= (1LL << 31)) return cudaErrorInvalidValue;
  unsigned char* p = static_cast<unsigned char*>(temp);
  int* keys_in = reinterpret_cast<int*>(p); p += align_up(sizeof(int) * (size_t)E);
  int* vals_in = reinterpret_cast<int*>(p); p += align_up(sizeof(int) * (size_t)E);
  p += align_up(sizeof(int) * (size_t)E);
  size_t cub_bytes = cub_sort_bytes(E);
  if ((size_t)(p - static_cast<unsigned char*>(temp)) + cub_bytes > temp_bytes) return cudaErrorInvalidValue;
  int bits = 1;
  while ((1LL << bits) < (long long)n_chunks * n_atoms + 1 && bits < 31) ++bits;
  chunk_key_kernel<<<(unsigned)((E + 255) / 256), 256, 0, s>>>(e_src, E, n_atoms, edge_ptr, n_chunks, keys_in, vals_in);
  return cub::DeviceRadixSort::SortPairs(p, cub_bytes, keys_in, keys, vals_in, perm, (int)E, 0, bits, s);
}

}  // namespace tace
