// Cell-list neighbour list for a batch of periodic (or partly periodic) structures.
//
// Semantics follow the reference's get_neighborhood (tace/dataset/neighbour_list.py:195-298,
// which wraps matscipy's "ijS" list): full list, edge vector r_target - r_source + S @ cell,
// strict |v| < cutoff evaluated in fp64, self pairs kept unless S = 0, no shift along
// non-periodic axes.  Cells narrower than the cutoff are handled by visiting several periodic
// images of the (single) bin along that axis.
//
// Atoms are binned per structure in fractional coordinates (bins at least cutoff / r wide, r
// bins searched on either side), sorted by bin with a stable radix sort, and every target atom
// walks its neighbouring bins in a fixed order, so the output order is deterministic: grouped
// by target, then by bin, then by source index.  The distance test uses the unwrapped input
// positions and explicit round-to-nearest multiplies/adds (no FMA contraction), so the edge set
// is bit-identical to a brute-force fp64 enumeration evaluated in the same order.
#include <cub/cub.cuh>
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/tace_b200.h"

namespace tace {
namespace {

struct GraphBins {
  double inv[9];   // frac = pos @ inv
  double cell[9];
  double fmin[3], fext[3];
  int nb[3], r[3], pbc[3];
  int bin_offset, n_bins;
};

__global__ void nl_setup_kernel(const double* __restrict__ pos, const double* __restrict__ lattice,
                                const uint8_t* __restrict__ pbc, const int* __restrict__ graph_ptr, double cutoff,
                                GraphBins* bins) {
  const int g = blockIdx.x;
  __shared__ double inv[9];
  __shared__ double smin[3][128], smax[3][128];
  const double* c = lattice + 9LL * g;
  if (threadIdx.x == 0) {
    const double det = c[0] * (c[4] * c[8] - c[5] * c[7]) - c[1] * (c[3] * c[8] - c[5] * c[6]) + c[2] * (c[3] * c[7] - c[4] * c[6]);
    const double id = 1.0 / det;
    inv[0] = (c[4] * c[8] - c[5] * c[7]) * id; inv[1] = (c[2] * c[7] - c[1] * c[8]) * id; inv[2] = (c[1] * c[5] - c[2] * c[4]) * id;
    inv[3] = (c[5] * c[6] - c[3] * c[8]) * id; inv[4] = (c[0] * c[8] - c[2] * c[6]) * id; inv[5] = (c[2] * c[3] - c[0] * c[5]) * id;
    inv[6] = (c[3] * c[7] - c[4] * c[6]) * id; inv[7] = (c[1] * c[6] - c[0] * c[7]) * id; inv[8] = (c[0] * c[4] - c[1] * c[3]) * id;
  }
  __syncthreads();
  double lo[3] = {1e300, 1e300, 1e300}, hi[3] = {-1e300, -1e300, -1e300};
  const int a0 = graph_ptr[g], a1 = graph_ptr[g + 1];
  for (int i = a0 + threadIdx.x; i < a1; i += blockDim.x) {
    const double x = pos[3LL * i], y = pos[3LL * i + 1], z = pos[3LL * i + 2];
    for (int k = 0; k < 3; ++k) {
      const double f = x * inv[k] + y * inv[3 + k] + z * inv[6 + k];
      lo[k] = fmin(lo[k], f); hi[k] = fmax(hi[k], f);
    }
  }
  for (int k = 0; k < 3; ++k) { smin[k][threadIdx.x] = lo[k]; smax[k][threadIdx.x] = hi[k]; }
  __syncthreads();
  for (int off = 64; off > 0; off >>= 1) {
    if (threadIdx.x < off)
      for (int k = 0; k < 3; ++k) {
        smin[k][threadIdx.x] = fmin(smin[k][threadIdx.x], smin[k][threadIdx.x + off]);
        smax[k][threadIdx.x] = fmax(smax[k][threadIdx.x], smax[k][threadIdx.x + off]);
      }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    GraphBins gb;
    for (int k = 0; k < 9; ++k) { gb.inv[k] = inv[k]; gb.cell[k] = c[k]; }
    const int n_atoms = a1 - a0;
    double width[3];
    for (int k = 0; k < 3; ++k) {
      // perpendicular height of the cell along axis k = 1 / |column k of inv|
      const double h = 1.0 / sqrt(inv[k] * inv[k] + inv[3 + k] * inv[3 + k] + inv[6 + k] * inv[6 + k]);
      gb.pbc[k] = pbc[3LL * g + k] ? 1 : 0;
      if (gb.pbc[k]) { gb.fmin[k] = 0.0; gb.fext[k] = 1.0; width[k] = h; }
      else {
        gb.fmin[k] = n_atoms ? smin[k][0] : 0.0;
        gb.fext[k] = n_atoms ? fmax(smax[k][0] - smin[k][0], 1e-12) : 1.0;
        width[k] = gb.fext[k] * h;
      }
      int nb = (int)floor(width[k] / cutoff);
      gb.nb[k] = nb < 1 ? 1 : (nb > 1024 ? 1024 : nb);
    }
    // keep the number of bins of a structure below ~2 per atom
    const long long cap = n_atoms > 0 ? 2LL * n_atoms : 1;
    while ((long long)gb.nb[0] * gb.nb[1] * gb.nb[2] > cap) {
      int k = 0;
      if (gb.nb[1] > gb.nb[k]) k = 1;
      if (gb.nb[2] > gb.nb[k]) k = 2;
      gb.nb[k] = (gb.nb[k] + 1) / 2;
    }
    for (int k = 0; k < 3; ++k) {
      const double bin_h = width[k] / gb.nb[k];
      int r = (int)ceil(cutoff / bin_h);
      if (r < 1) r = 1;
      if (!gb.pbc[k] && r > gb.nb[k] - 1) r = gb.nb[k] - 1;
      gb.r[k] = r;
    }
    gb.n_bins = gb.nb[0] * gb.nb[1] * gb.nb[2];
    gb.bin_offset = 0;
    bins[g] = gb;
  }
}

__global__ void nl_offsets_kernel(GraphBins* bins, int n_graphs, int* total) {
  if (blockIdx.x || threadIdx.x) return;
  int acc = 0;
  for (int g = 0; g < n_graphs; ++g) { bins[g].bin_offset = acc; acc += bins[g].n_bins; }
  *total = acc;
}

__global__ void nl_bin_kernel(const double* __restrict__ pos, const GraphBins* __restrict__ bins,
                              const int* __restrict__ graph_ptr, int n_graphs, int n_atoms, int* keys, int* vals, int* img) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_atoms) return;
  int lo = 0, hi = n_graphs;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (graph_ptr[mid] <= i) lo = mid; else hi = mid; }
  const GraphBins& gb = bins[lo];
  const double x = pos[3LL * i], y = pos[3LL * i + 1], z = pos[3LL * i + 2];
  int b[3];
  for (int k = 0; k < 3; ++k) {
    const double f = x * gb.inv[k] + y * gb.inv[3 + k] + z * gb.inv[6 + k];
    int fl = 0;
    double t;
    if (gb.pbc[k]) { const double ff = floor(f); fl = (int)ff; t = f - ff; }
    else t = (f - gb.fmin[k]) / gb.fext[k];
    int bk = (int)(t * gb.nb[k]);
    bk = bk < 0 ? 0 : (bk >= gb.nb[k] ? gb.nb[k] - 1 : bk);
    b[k] = bk;
    img[3LL * i + k] = fl;
  }
  keys[i] = gb.bin_offset + (b[0] * gb.nb[1] + b[1]) * gb.nb[2] + b[2];
  vals[i] = i;
}

__global__ void nl_cell_start_kernel(const int* __restrict__ sorted_keys, int n_keys, int* cell_start, int n_cells) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c > n_cells) return;
  int lo = 0, hi = n_keys;
  while (lo < hi) { const int mid = (lo + hi) >> 1; if (sorted_keys[mid] < c) lo = mid + 1; else hi = mid; }
  cell_start[c] = lo;
}

__device__ __forceinline__ int floordiv(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }

// FILL = false: counts[i] = number of sources of target i; FILL = true: write them at row_ptr[i].
// One warp per target atom: every lane takes one neighbouring bin (bins are visited in the fixed order d0, d1, d2 of
// the offsets), counts the sources of its bin that lie inside the cutoff, an exclusive scan over the lanes turns the
// counts into output positions, and the lane tests its bin again to write.  The output order (by bin, then by sorted
// source position) does not depend on the lane assignment, so it is deterministic.
template <bool FILL>
__global__ void __launch_bounds__(128) nl_search_kernel(const double* __restrict__ pos, const GraphBins* __restrict__ bins,
                                 const int* __restrict__ graph_ptr, int n_graphs, int n_atoms, double cutoff,
                                 const int* __restrict__ keys_of_atom, const int* __restrict__ sorted_atoms,
                                 const int* __restrict__ cell_start, const int* __restrict__ img, int* counts,
                                 const int64_t* __restrict__ row_ptr, int64_t n_edges, int64_t* edge_index, int32_t* shifts) {
  const int i = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (i >= n_atoms) return;  // whole warps leave together
  int lo = 0, hi = n_graphs;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (graph_ptr[mid] <= i) lo = mid; else hi = mid; }
  const GraphBins& gb = bins[lo];
  const double c2 = __dmul_rn(cutoff, cutoff);
  const double xi = pos[3LL * i], yi = pos[3LL * i + 1], zi = pos[3LL * i + 2];
  const int key = keys_of_atom[i] - gb.bin_offset;
  const int b2 = key % gb.nb[2], b1 = (key / gb.nb[2]) % gb.nb[1], b0 = key / (gb.nb[2] * gb.nb[1]);
  const int fi0 = img[3LL * i], fi1 = img[3LL * i + 1], fi2 = img[3LL * i + 2];
  const int w1 = 2 * gb.r[1] + 1, w2 = 2 * gb.r[2] + 1;
  const int n_cells = (2 * gb.r[0] + 1) * w1 * w2;
  int64_t out = FILL ? row_ptr[i] : 0;
  int count = 0;
  for (int cb = 0; cb < n_cells; cb += 32) {
    const int c = cb + lane;
    int k_beg = 0, k_end = 0, s0 = 0, s1 = 0, s2 = 0;
    if (c < n_cells) {
      const int d0 = c / (w1 * w2) - gb.r[0], d1 = (c / w2) % w1 - gb.r[1], d2 = c % w2 - gb.r[2];
      int c0 = b0 + d0, c1 = b1 + d1, c2i = b2 + d2;
      bool inside = true;
      if (gb.pbc[0]) { s0 = floordiv(c0, gb.nb[0]); c0 -= s0 * gb.nb[0]; } else if (c0 < 0 || c0 >= gb.nb[0]) inside = false;
      if (gb.pbc[1]) { s1 = floordiv(c1, gb.nb[1]); c1 -= s1 * gb.nb[1]; } else if (c1 < 0 || c1 >= gb.nb[1]) inside = false;
      if (gb.pbc[2]) { s2 = floordiv(c2i, gb.nb[2]); c2i -= s2 * gb.nb[2]; } else if (c2i < 0 || c2i >= gb.nb[2]) inside = false;
      if (inside) {
        const int cell = gb.bin_offset + (c0 * gb.nb[1] + c1) * gb.nb[2] + c2i;
        k_beg = cell_start[cell]; k_end = cell_start[cell + 1];
      }
    }
    // wrapped image (s0,s1,s2) of source j seen from target i:  r_j - r_i + S' @ cell with S' = s - fl_j + fl_i;
    // the edge (source j -> target i) carries shift S = -S'.
    auto test = [&](int k, int& j, int& S0, int& S1, int& S2) -> bool {
      j = sorted_atoms[k];
      S0 = -(s0 - img[3LL * j] + fi0); S1 = -(s1 - img[3LL * j + 1] + fi1); S2 = -(s2 - img[3LL * j + 2] + fi2);
      if (j == i && S0 == 0 && S1 == 0 && S2 == 0) return false;
      const double t0 = __dadd_rn(__dadd_rn(__dmul_rn((double)S0, gb.cell[0]), __dmul_rn((double)S1, gb.cell[3])), __dmul_rn((double)S2, gb.cell[6]));
      const double t1 = __dadd_rn(__dadd_rn(__dmul_rn((double)S0, gb.cell[1]), __dmul_rn((double)S1, gb.cell[4])), __dmul_rn((double)S2, gb.cell[7]));
      const double t2 = __dadd_rn(__dadd_rn(__dmul_rn((double)S0, gb.cell[2]), __dmul_rn((double)S1, gb.cell[5])), __dmul_rn((double)S2, gb.cell[8]));
      const double dx = __dadd_rn(__dadd_rn(xi, -pos[3LL * j]), t0);
      const double dy = __dadd_rn(__dadd_rn(yi, -pos[3LL * j + 1]), t1);
      const double dz = __dadd_rn(__dadd_rn(zi, -pos[3LL * j + 2]), t2);
      const double dsq = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
      return dsq < c2;
    };
    int n = 0, j, S0, S1, S2;
    for (int k = k_beg; k < k_end; ++k) n += test(k, j, S0, S1, S2) ? 1 : 0;
    int incl = n;  // inclusive scan over the lanes
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (FILL && n > 0) {
      int64_t at = out + (incl - n);
      for (int k = k_beg; k < k_end; ++k) {
        if (test(k, j, S0, S1, S2)) {
          if (at < n_edges) {
            edge_index[at] = j;
            edge_index[n_edges + at] = i;
            shifts[3 * at] = S0; shifts[3 * at + 1] = S1; shifts[3 * at + 2] = S2;
          }
          ++at;
        }
      }
    }
    out += total;
    count += total;
  }
  if (!FILL && lane == 0) counts[i] = count;
}

size_t nl_workspace_bytes(int n_atoms, int n_graphs) {
  auto al = [](size_t x) { return (x + 255) & ~size_t(255); };
  const int max_cells = 2 * n_atoms + n_graphs + 1;
  size_t cub_bytes = 0;
  if (n_atoms > 0)
    cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const int*)nullptr, (int*)nullptr, (const int*)nullptr, (int*)nullptr, n_atoms);
  return al(sizeof(GraphBins) * n_graphs) + al(sizeof(int)) + 4 * al(sizeof(int) * (size_t)n_atoms) +
         al(sizeof(int) * 3 * (size_t)n_atoms) + al(sizeof(int) * (size_t)(max_cells + 1)) + al(cub_bytes) + 256;
}

int nl_run(bool fill, const double* pos, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr, int32_t n_graphs,
           int64_t n_atoms64, double cutoff, int32_t* counts, const int64_t* row_ptr, int64_t n_edges, int64_t* edge_index,
           int32_t* shifts, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (!pos || !lattice || !pbc || !graph_ptr || n_graphs <= 0 || n_atoms64 < 0 || !(cutoff > 0.0)) return TACE_ERR_INVALID_ARGUMENT;
  if (n_atoms64 >= (1LL << 30)) return TACE_ERR_CAPACITY;
  if (fill ? (!row_ptr || (n_edges > 0 && (!edge_index || !shifts))) : !counts) return TACE_ERR_INVALID_ARGUMENT;
  const int n_atoms = (int)n_atoms64;
  if (n_atoms == 0) return TACE_OK;
  if (!workspace) return TACE_ERR_INVALID_ARGUMENT;
  const int max_cells = 2 * n_atoms + n_graphs + 1;
  size_t cub_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const int*)nullptr, (int*)nullptr, (const int*)nullptr, (int*)nullptr, n_atoms);
  auto al = [](size_t x) { return (x + 255) & ~size_t(255); };
  // the caller's scratch, cut up from its first 256-byte boundary
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  const size_t lead = (size_t)(base - static_cast<unsigned char*>(workspace));
  if (workspace_bytes < lead || workspace_bytes - lead + 256 < nl_workspace_bytes(n_atoms, n_graphs)) return TACE_ERR_CAPACITY;
  unsigned char* p = base;
  GraphBins* bins = reinterpret_cast<GraphBins*>(p); p += al(sizeof(GraphBins) * n_graphs);
  int* total = reinterpret_cast<int*>(p); p += al(sizeof(int));
  int* keys = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)n_atoms);
  int* vals = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)n_atoms);
  int* keys_sorted = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)n_atoms);
  int* atoms_sorted = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)n_atoms);
  int* img = reinterpret_cast<int*>(p); p += al(sizeof(int) * 3 * (size_t)n_atoms);
  int* cell_start = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)(max_cells + 1));
  void* cub_temp = p;

  nl_setup_kernel<<<n_graphs, 128, 0, s>>>(pos, lattice, pbc, graph_ptr, cutoff, bins);
  nl_offsets_kernel<<<1, 1, 0, s>>>(bins, n_graphs, total);
  const int ab = (n_atoms + 127) / 128;
  const unsigned wb = (unsigned)((n_atoms + 3) / 4);  // search kernels: one warp per atom, four warps per block
  nl_bin_kernel<<<ab, 128, 0, s>>>(pos, bins, graph_ptr, n_graphs, n_atoms, keys, vals, img);
  cudaError_t err = cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, keys, keys_sorted, vals, atoms_sorted, n_atoms, 0, 32, s);
  if (err == cudaSuccess) {
    nl_cell_start_kernel<<<(max_cells + 128) / 128, 128, 0, s>>>(keys_sorted, n_atoms, cell_start, max_cells);
    if (fill)
      nl_search_kernel<true><<<wb, 128, 0, s>>>(pos, bins, graph_ptr, n_graphs, n_atoms, cutoff, keys, atoms_sorted, cell_start, img,
                                                nullptr, row_ptr, n_edges, edge_index, shifts);
    else
      nl_search_kernel<false><<<wb, 128, 0, s>>>(pos, bins, graph_ptr, n_graphs, n_atoms, cutoff, keys, atoms_sorted, cell_start, img,
                                                 counts, nullptr, 0, nullptr, nullptr);
    err = cudaGetLastError();
  }
  return err == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

// ---- neighbour list without any allocation -------------------------------------------------------
// Scratch for tace_nl_build_noalloc lives in this file-scope device array (2 MiB per GPU that loads
// the library, held until the process exits).  In host code the name `nl_static_scratch` is only a
// handle for the runtime, not a device address: the address is looked up once per device with
// cudaGetSymbolAddress and that pointer is what the kernels receive.
constexpr int kNoAllocMaxAtoms = 16384;
constexpr int kNoAllocMaxGraphs = 1024;
constexpr size_t kNoAllocScratchBytes = size_t(2) << 20;
static __device__ __align__(256) unsigned char nl_static_scratch[kNoAllocScratchBytes];

// row_ptr[0] = 0, row_ptr[i + 1] = counts[0] + ... + counts[i]; one block, any n
__global__ void nl_scan_counts_kernel(const int* __restrict__ counts, int n, int64_t* row_ptr) {
  __shared__ long long part[1024];
  __shared__ long long carry;
  if (threadIdx.x == 0) { carry = 0; row_ptr[0] = 0; }
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    part[threadIdx.x] = i < n ? counts[i] : 0;
    __syncthreads();
    for (int off = 1; off < (int)blockDim.x; off <<= 1) {  // inclusive Hillis-Steele scan of this chunk
      const long long add = (int)threadIdx.x >= off ? part[threadIdx.x - off] : 0;
      __syncthreads();
      part[threadIdx.x] += add;
      __syncthreads();
    }
    if (i < n) row_ptr[i + 1] = carry + part[threadIdx.x];
    __syncthreads();
    if (threadIdx.x == 0) carry += part[blockDim.x - 1];
    __syncthreads();
  }
}

int nl_build_noalloc(const double* pos, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr, int32_t n_graphs,
                     int64_t n_atoms64, double cutoff, int64_t max_edges, int64_t* row_ptr, int64_t* edge_index, int32_t* shifts,
                     cudaStream_t s) {
  if (!pos || !lattice || !pbc || !graph_ptr || !row_ptr || n_graphs <= 0 || n_atoms64 < 0 || max_edges < 0 || !(cutoff > 0.0) ||
      (max_edges > 0 && (!edge_index || !shifts)))
    return TACE_ERR_INVALID_ARGUMENT;
  if (n_atoms64 > kNoAllocMaxAtoms || n_graphs > kNoAllocMaxGraphs) return TACE_ERR_CAPACITY;
  const int n_atoms = (int)n_atoms64;
  // one-time, per-device lookup of the scratch array's device address (with that device current)
  constexpr int kMaxDevices = 64;
  static unsigned char* scratch_of_device[kMaxDevices] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TACE_ERR_NO_DEVICE;
  if (!scratch_of_device[dev]) {
    unsigned char* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, nl_static_scratch) != cudaSuccess || !ptr) return TACE_ERR_CUDA;
    scratch_of_device[dev] = ptr;
  }
  unsigned char* p = scratch_of_device[dev];
  unsigned char* const end = p + kNoAllocScratchBytes;
  auto al = [](size_t x) { return (x + 255) & ~size_t(255); };
  const int max_cells = 2 * n_atoms + n_graphs + 1;
  GraphBins* bins = reinterpret_cast<GraphBins*>(p); p += al(sizeof(GraphBins) * n_graphs);
  int* total = reinterpret_cast<int*>(p); p += al(sizeof(int));
  int* keys = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)(n_atoms + 1));
  int* vals = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)(n_atoms + 1));
  int* keys_sorted = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)(n_atoms + 1));
  int* atoms_sorted = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)(n_atoms + 1));
  int* img = reinterpret_cast<int*>(p); p += al(sizeof(int) * 3 * (size_t)(n_atoms + 1));
  int* cell_start = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)(max_cells + 1));
  int* counts = reinterpret_cast<int*>(p); p += al(sizeof(int) * (size_t)(n_atoms + 1));
  size_t cub_bytes = 0;
  if (n_atoms > 0)
    cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const int*)nullptr, (int*)nullptr, (const int*)nullptr, (int*)nullptr, n_atoms);
  void* cub_temp = p;
  if (p + cub_bytes > end) return TACE_ERR_CAPACITY;

  if (n_atoms == 0) {
    nl_scan_counts_kernel<<<1, 32, 0, s>>>(counts, 0, row_ptr);
    return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
  }
  nl_setup_kernel<<<n_graphs, 128, 0, s>>>(pos, lattice, pbc, graph_ptr, cutoff, bins);
  nl_offsets_kernel<<<1, 1, 0, s>>>(bins, n_graphs, total);
  const int ab = (n_atoms + 127) / 128;
  const unsigned wb = (unsigned)((n_atoms + 3) / 4);  // search kernels: one warp per atom, four warps per block
  nl_bin_kernel<<<ab, 128, 0, s>>>(pos, bins, graph_ptr, n_graphs, n_atoms, keys, vals, img);
  if (cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, keys, keys_sorted, vals, atoms_sorted, n_atoms, 0, 32, s) != cudaSuccess)
    return TACE_ERR_CUDA;
  nl_cell_start_kernel<<<(max_cells + 128) / 128, 128, 0, s>>>(keys_sorted, n_atoms, cell_start, max_cells);
  nl_search_kernel<false><<<wb, 128, 0, s>>>(pos, bins, graph_ptr, n_graphs, n_atoms, cutoff, keys, atoms_sorted, cell_start, img,
                                             counts, nullptr, 0, nullptr, nullptr);
  nl_scan_counts_kernel<<<1, 1024, 0, s>>>(counts, n_atoms, row_ptr);
  nl_search_kernel<true><<<wb, 128, 0, s>>>(pos, bins, graph_ptr, n_graphs, n_atoms, cutoff, keys, atoms_sorted, cell_start, img,
                                            nullptr, row_ptr, max_edges, edge_index, shifts);
  return cudaGetLastError() == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

}  // namespace
}  // namespace tace

extern "C" {

int tace_nl_build_noalloc(const double* positions, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr,
                          int32_t n_graphs, int64_t n_atoms, double cutoff, int64_t max_edges, int64_t* row_ptr,
                          int64_t* edge_index, int32_t* edge_shifts, tace_stream_t stream) {
  return tace::nl_build_noalloc(positions, lattice, pbc, graph_ptr, n_graphs, n_atoms, cutoff, max_edges, row_ptr, edge_index,
                                edge_shifts, static_cast<cudaStream_t>(stream));
}

int tace_nl_workspace_bytes(int64_t n_atoms, int32_t n_graphs, size_t* bytes) {
  if (!bytes || n_atoms < 0 || n_graphs <= 0) return TACE_ERR_INVALID_ARGUMENT;
  if (n_atoms >= (1LL << 30)) return TACE_ERR_CAPACITY;
  *bytes = tace::nl_workspace_bytes((int)n_atoms, n_graphs);
  return TACE_OK;
}

int tace_nl_count(const double* positions, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr,
                  int32_t n_graphs, int64_t n_atoms, double cutoff, int32_t* counts, void* workspace, size_t workspace_bytes,
                  tace_stream_t stream) {
  return tace::nl_run(false, positions, lattice, pbc, graph_ptr, n_graphs, n_atoms, cutoff, counts, nullptr, 0, nullptr, nullptr,
                      workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int tace_nl_fill(const double* positions, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr,
                 int32_t n_graphs, int64_t n_atoms, double cutoff, const int64_t* row_ptr, int64_t n_edges,
                 int64_t* edge_index, int32_t* edge_shifts, void* workspace, size_t workspace_bytes, tace_stream_t stream) {
  return tace::nl_run(true, positions, lattice, pbc, graph_ptr, n_graphs, n_atoms, cutoff, nullptr, row_ptr, n_edges, edge_index,
                      edge_shifts, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
