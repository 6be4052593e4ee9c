// Internal launcher interface between the engine (engine.cu) and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "tace_math.cuh"

namespace tace {

constexpr int kMaxLayers = 4;


// ---- interaction tensor product (tp_kernels.cu) ---------------------------------------------
// Message passing m_i = sum_{e: target(e) = i} sum_p w[e,p,c] (x[source(e)] (x) Y[e])_p, its
// transpose with respect to the source features, and the gradients with respect to the
// per-edge weights and angular features.  Follows O3ScatterTensorProduct.forward
// (tace/models/_e3nn/fused.py:259-271); edges are grouped by target (forward, edge gradients)
// or by source (source gradients) so every sum is a segmented reduction without atomics.
template <typename T>
struct TPArgs {
  int L, scalar_src, C;  // L: rank of Y and of the messages; scalar_src: the source is one scalar block (first layer)
  int Lin;               // rank of the source features when !scalar_src (1..L)
  int n_seg;          // number of target atoms = thread blocks (per output group)
  const int* rowptr;  // [n_seg+1] CSR over the edges of each target (edges are target-sorted)
  // Partial passes (target atoms that see no ghost source while the ghost rows of x are still in flight, the others
  // afterwards): with row_ids the thread blocks of part 0 work on the targets row_ids[0 .. *row_split), those of part 1 on
  // row_ids[*row_split .. n_seg); both are launched with n_seg blocks, the surplus blocks return at once
  const int* row_ids;    // [n_seg] or nullptr (then block i works on target i)
  const int* row_split;  // device word
  int row_part;
  const int* e_src;   // [E] source atom of each edge
  const T* Y;         // [E][D] spherical harmonics of each edge
  const T* W;         // [E][NP*C] per-edge path weights
  const T* x;         // [N][NX][C] source features
  T* M;               // forward output [n_seg][NM][C]
  const T* gM;        // [n_seg][NM][C] gradient of the messages
  T* dW;              // backward output [E][NP*C] (may alias W)
  T* dY;              // backward output [E][D]
  int accumulate_dY;  // add into dY instead of overwriting
  T* dxe;             // backward output [E][NX][C]: per-edge gradient of the source features (full source only)
  // radial_basis.apply_cutoff = False: the path weights are env[e] * W[e, :]; the backward pass stores env[e] * dW and
  // the per-edge sum of dW * W (gradient with respect to the envelope) in denv
  const T* env;       // [E] or nullptr
  T* denv;            // [E] or nullptr
  int accumulate_denv;
  long long e_base;   // W, dW and dxe hold the rows of edges [e_base, ...) only (edge-chunked passes); Y, dY, e_src are whole
  // Tabulated path weights (models with the identity edge update, where the radial MLP's output is a function of the
  // edge length alone): rtab [rt_K][NP*C][4] = (W, h dW/dd) at both ends of the interval [k h, (k + 1) h], read with cubic
  // Hermite interpolation instead of W; the backward pass then writes no dW and adds sum_{p,c} dW * dW/dd into ddlen.
  const T* rtab;      // nullptr: per-edge weights W / dW as above
  int rt_K;           // number of intervals
  T rt_inv_h;         // 1 / knot spacing
  const T* dlen;      // [E] edge lengths
  T* ddlen;           // [E] dE/d(edge length), backward
  int accumulate_ddlen;
};
template <typename T> cudaError_t launch_tp_fwd(const TPArgs<T>& a, cudaStream_t s);
template <typename T> cudaError_t launch_tp_bwd(const TPArgs<T>& a, cudaStream_t s);
// gx[b] = sum of dxe over the edges whose source is b (edges listed by perm within rowptr_src segments)
// for the source atoms [first_atom, first_atom + n_atoms)
template <typename T> cudaError_t launch_segment_sum_rows(const T* dxe, const int* rowptr_src, const int* perm_src, T* gx,
                                                          int first_atom, int n_atoms, int row_len, cudaStream_t s);
// Edge-chunked variant: positions [k0, k1) of the (chunk, source)-sorted edge list belong to one chunk whose dxe rows start
// at edge k0; every run of equal keys is summed in list order and ADDED to gx[key - key_base] (runs of one chunk have
// distinct sources, chunks are processed one after another, so the sum order is fixed).
template <typename T> cudaError_t launch_chunk_src_sum(const T* dxe_chunk, const int* keys, const int* perm, long long k0,
                                                       long long k1, long long key_base, T* gx, int row_len, cudaStream_t s);

// ---- per-atom element-wise kernels (node_kernels.cu) -----------------------------------------
// x0[n][c] = table[species[n]][c]
template <typename T> cudaError_t launch_species_gather(const T* table, const int* species, T* out, int n, int C, cudaStream_t s);
// gate (tace/models/_e3nn/nonlinear.py:125-135): Gt = [(L+1)C gates | D*C gated] per atom.
// Third-order product basis (correlation 3): B3 = (A x A) x A with B2 the full second-order basis (ranks <= L).
// launch_pb3_bwd adds the gradients into gB2 and gA.
template <typename T> cudaError_t launch_pb3_fwd(const T* A, const T* B2, T* B3, int n, int L, int Lout, int C, cudaStream_t s);
template <typename T> cudaError_t launch_pb3_bwd(const T* A, const T* B2, const T* gB3, T* gB2, T* gA, int n, int L, int Lout, int C,
                                                 cudaStream_t s);
// m0: 1 = every rank (l = 0 included) scaled by a sigmoid gate; 0 = scalars through the normalised SiLU, ranks >= 1 gated
template <typename T> cudaError_t launch_gate_fwd(const T* Gt, T* a, int n, int L, int C, int m0, cudaStream_t s);
template <typename T> cudaError_t launch_gate_bwd(const T* Gt, const T* ga, T* gGt, int n, int L, int C, int m0, cudaStream_t s);
// product basis A (x) A (tace/models/_e3nn/prod.py:242-256, fused.py:90-95)
// L: rank of A; Lout: highest output rank, or < 0 for scalar outputs only (the last layer)
template <typename T> cudaError_t launch_pb_fwd(const T* A, T* B2, int n, int L, int Lout, int C, cudaStream_t s);
template <typename T> cudaError_t launch_pb_bwd(const T* A, const T* gB2, T* gA, int n, int L, int Lout, int C, cudaStream_t s);
// gated bilinear product (product_basis.nonlinear = silu_bilineargate): XY [n][D][2C] holds both factors (channels [0, C) /
// [C, 2C)), Zg [n][NP][C] the gate pre-activations; B2 = silu(Zg) * (x (x) [y, 1]).  bwd: gXY[.., :C] += , gXY[.., C:] = ,
// gZg = (gradients of the pre-activations)
template <typename T> cudaError_t launch_pbl_fwd(const T* XY, const T* Zg, T* B2, int n, int L, int Lout, int C, cudaStream_t s);
template <typename T> cudaError_t launch_pbl_bwd(const T* XY, const T* Zg, const T* gB2, T* gXY, T* gZg, int n, int L, int Lout, int C,
                                                cudaStream_t s);
// read-out C -> H -> 1 with scaled SiLU, per-species scale, isolated-atom masking, atomic energies
// (tace/models/_e3nn/readout.py:72-84, tace/models/blocks.py:250-273,332-379, _e3nn/tace.py:361-417).
template <typename T>
struct ReadoutArgs {
  const T* h;        // [n][hs] scalar channels at offset 0, stride hs
  long long hs;
  const T* W1;       // [C][H]
  const T* W2;       // [H]
  const T* scale;    // [n_el]
  const T* e0;       // [n_el]
  const int* species;
  const int* atom_graph;  // [n] graph of each atom
  const int* graph_ptr;   // [B+1]
  const int* rowptr_dst;  // [n+1] to count a graph's edges
  T* node_energy;    // [n] or nullptr (E0 + scaled read-out)
  T* e_scaled;       // [n] scaled read-out without E0 (summed per graph together with E0)
  T* gh;             // [n][C] d(sum E)/dh, or nullptr
  int n, C, H;
  // linear read-outs of earlier layers (use_alllayer): e += sum_c extra_h[t][i * extra_hs[t] + c] * extra_w[t][c]
  int n_extra;
  const T* extra_h[kMaxLayers]; long long extra_hs[kMaxLayers]; const T* extra_w[kMaxLayers];
  T* factor;         // [n] d(node energy)/d(read-out sum): the species scale, 0 for isolated atoms; or nullptr
  // multi-head read-out (tace/models/_e3nn/readout.py:18-33): W1 [n_fid][C][H], W2 [n_fid][H], scale / e0 [n_fid][n_el],
  // extra_w [n_fid][C]; fidelity[g] is the head of graph g (nullptr: head 0)
  const int* fidelity; int n_el;
  // pair repulsion per atom (launch_zbl_fwd) or nullptr; added before the species scale, or after it when zbl_after
  const T* zbl; int zbl_after;
};
// gh[i * hs + c] += factor[i] * w[f_i * C + c]: gradient of an earlier layer's linear read-out (f_i = head of atom i's graph)
template <typename T> cudaError_t launch_readout_linear_bwd(T* gh, long long hs, const T* factor, const T* w, const int* atom_graph,
                                                           const int* fidelity, int n, int C, cudaStream_t s);
// ZBL pair repulsion (tace/models/radial.py:788-874): v_e = 0.5 * 14.3996 Zu Zv / d * phi(d / a) * envelope(d, rcov_u + rcov_v)
// with a = par[0] / (Zu^par[1] + Zv^par[1]).  Forward: node[i] = sum of v_e over the edges into i (target-sorted CSR);
// backward: ddlen[e] += factor[target(e)] * dv_e/dd (factor == nullptr: 1).
template <typename T>
struct ZblArgs {
  const int* rowptr_dst; const int* e_src; const int* e_dst; const int* species;
  const T* dlen; const T* z; const T* rcov; const T* par; int p;
  int n; long long E;
  T* node; const T* factor; T* ddlen;
};
// Learned edge density replacing the constant 1/avg_num_neighbors (atomic_basis.scatter_norm = density,
// tace/models/_e3nn/inter.py:102-110,249-260): rho_e = tanh(y_e^2) [* envelope], y_e = silu(radial(d_e) A0 + b0) . w1 + b1,
// density_i = beta * sum_{e -> i} rho_e + alpha (1e-9 where exactly 0), messages / density_i.
// fwd: inv_density[i]; bwd: ddlen[e] += gdens[target(e)] * beta * d rho_e / d d.  ab = {alpha, beta}.
template <typename T>
struct DensityArgs {
  const int* rowptr_dst; const int* e_dst; const T* dlen; RadialParams<T> rp;
  const T* A0; const T* b0; const T* w1; const T* b1; const T* ab;
  int use_env;  // multiply rho_e by the envelope (apply_cutoff = False with scatter_norm = density)
  int n; long long E;
  T* inv_density; const T* gdens; T* ddlen;
};
template <typename T> cudaError_t launch_density_fwd(const DensityArgs<T>& a, cudaStream_t s);
template <typename T> cudaError_t launch_density_bwd(const DensityArgs<T>& a, cudaStream_t s);
// x[i, :width] *= scale[i] (rows `stride` elements apart)
template <typename T> cudaError_t launch_scale_rows(T* x, const T* scale, long long n, int width, long long stride, cudaStream_t s);
// gdens[i] = -inv[i] * sum_k gx[i, k] * x[i, k] (0 where the density was replaced by 1e-9), then gx[i, :width] *= inv[i]
template <typename T> cudaError_t launch_density_node_bwd(T* gx, const T* x, const T* inv, T* gdens, long long n, int width,
                                                         long long stride, cudaStream_t s);
template <typename T> cudaError_t launch_zbl_fwd(const ZblArgs<T>& a, cudaStream_t s);
template <typename T> cudaError_t launch_zbl_bwd(const ZblArgs<T>& a, cudaStream_t s);
template <typename T> cudaError_t launch_readout(const ReadoutArgs<T>& a, cudaStream_t s);
// energy[g] = sum_{i in g} (e0[species_i] + e_scaled[i])
// slices per graph of the per-graph energy sum: one per 8 192 atoms of the average graph (1 for batches of small graphs,
// 64 at most); `partial` holds n_graphs * slices values (needed when slices > 1)
inline int graph_energy_slices(long long n_atoms, int n_graphs) {
  if (n_graphs <= 0) return 1;
  const long long per = n_atoms / n_graphs / 8192;
  return per < 1 ? 1 : (per > 64 ? 64 : (int)per);
}
template <typename T> cudaError_t launch_graph_energy(const T* e_scaled, const T* e0, const int* species, const int* graph_ptr,
                                                      const int* fidelity, int n_el, T* energy, int n_graphs, long long n_atoms,
                                                      T* partial, cudaStream_t s);
template <typename T> cudaError_t launch_fill_zero(T* p, long long n, cudaStream_t s);
// dst[i] = src[perm[i]] (gather) / dst[perm[i]] = src[i] (scatter), rows of row_len elements
template <typename T> cudaError_t launch_gather_rows(const T* src, const int* perm, T* dst, long long n, int row_len, cudaStream_t s);
template <typename T> cudaError_t launch_scatter_rows(const T* src, const int* perm, T* dst, long long n, int row_len, cudaStream_t s);
template <typename T> cudaError_t launch_add_inplace(T* dst, const T* src, long long n, cudaStream_t s);
// dst[i, :width] += src[i, :width], rows dst_stride / src_stride elements apart
template <typename T> cudaError_t launch_add_rows(T* dst, long long dst_stride, const T* src, long long src_stride, long long n, int width,
                                                 cudaStream_t s);

// ---- per-edge kernels (edge_kernels.cu) -------------------------------------------------------
template <typename T>
struct MlpWeights {
  const T* A0; const T* A1; const T* A2; const T* A1t; const T* A2t;
  const T* b0;       // [64] bias of the first layer, or nullptr
  // edge_update "element2" (tace/models/_e3nn/edge.py:237-257): the species embeddings of both ends are concatenated to
  // the radial features, i.e. they add a species-dependent row to the first pre-activation: tables [n_el][64] or nullptr
  const T* tbl_dst; const T* tbl_src;
};
template <typename T>
struct EdgeArgs {
  int L, n_layers;
  long long E;
  const int* e_src; const int* e_dst; const int* e_orig;  // target-sorted edges; e_orig = caller's edge id
  const T* positions;    // [N][3] or nullptr
  const T* lattice;      // [B][3][3]
  const int* atom_graph; // [N]
  const T* shifts;       // [E][3] caller order, or nullptr
  const T* edge_vector;  // [E][3] caller order, or nullptr
  RadialParams<T> rp;
  MlpWeights<T> mlp[kMaxLayers];
  T* dlen;               // [E] edge length |v| + 1e-9
  T* ddlen;              // [E] dE/d(edge length) through the radial branch (backward)
  T* vec;                // [E][3] edge vectors (target-sorted order)
  T* Y;                  // [E][D]
  T* Z1[kMaxLayers];     // [E][64] pre-activation of the first hidden layer of each layer's radial MLP
  T* H1[kMaxLayers];     // [E][64] its activation silu(Z1), written by launch_edge_mlp_in as well
  const T* dH1[kMaxLayers];  // [E][64] gradient of the first hidden activation (backward)
  int accumulate_ddlen;  // launch_edge_mlp_out adds into ddlen instead of overwriting (layer-by-layer passes)
  const int* species;    // [N] (element-dependent edge update), or nullptr
  T* env;                // [E] envelope values, written by launch_edge_fwd when the cutoff is applied after the MLP
  const T* denv;         // [E] dE/d(envelope) from the tensor-product backward passes (same case), or nullptr
  int add_denv;          // this launch_edge_mlp_out call adds the envelope term to ddlen
  const T* gvec_extra;   // [E][3] added to dE/d(edge vector) by launch_edge_bwd (gradient through the TECE edge frames), or nullptr
  int dz1_given;         // dH1 holds dE/d(first pre-activation) already (LayerNorm models): launch_edge_mlp_out applies no silu'
  // backward
  const T* dY;           // [E][D]
  T* g;                  // [E][3] dE/d(edge vector), target-sorted order
  T* edge_forces;        // [E][3] caller order, or nullptr
};
template <typename T> cudaError_t launch_edge_fwd(const EdgeArgs<T>& a, cudaStream_t s);
template <typename T> cudaError_t launch_edge_bwd(const EdgeArgs<T>& a, cudaStream_t s);
// radial MLP: first layer (8 -> 64) forward / backward per edge; the 64 -> 64 layers are GEMMs
template <typename T> cudaError_t launch_edge_mlp_in(const EdgeArgs<T>& a, cudaStream_t s);
template <typename T> cudaError_t launch_edge_mlp_out(const EdgeArgs<T>& a, cudaStream_t s);
template <typename T> cudaError_t launch_silu(const T* in, T* out, long long n, cudaStream_t s);           // out = silu(in)
template <typename T> cudaError_t launch_silu_grad_mul(T* g, const T* z, long long n, cudaStream_t s);     // g *= silu'(z)
// rows of 64 features: h = silu(LayerNorm(z) * gamma + beta); g <- dE/dz from g = dE/dh (statistics recomputed from z)
template <typename T> cudaError_t launch_ln_silu_fwd(const T* z, const T* gamma, const T* beta, T* h, long long rows, cudaStream_t s);
template <typename T> cudaError_t launch_ln_silu_bwd(T* g, const T* z, const T* gamma, const T* beta, long long rows, cudaStream_t s);

// forces[i] = -(sum_{e: target = i} g_e - sum_{e: source = i} g_e); per-atom virial rows
// w[i] = sum_{e: target = i} v_e (x) g_e (tace/models/adapter.py:106-116, utils.py:50-79).
template <typename T>
struct ForceArgs {
  int n_atoms, n_local;
  const int* rowptr_dst; const int* rowptr_src; const int* perm_src;
  const T* g; const T* vec;
  T* forces;       // [n_atoms][3] or nullptr
  T* atom_virial;  // [n_local][9] or nullptr
};
template <typename T> cudaError_t launch_forces(const ForceArgs<T>& a, cudaStream_t s);
// virials[g] = -sym(sum_i w[i]); stress = -virials / |det lattice| with |stress| >= 1e10 zeroed
template <typename T> cudaError_t launch_graph_virial(const T* atom_virial, const int* graph_ptr, const T* lattice, T* virials,
                                                     T* stress, int n_graphs, cudaStream_t s);

// ---- graph preparation (graph_kernels.cu) ------------------------------------------------------
struct GraphPrepArgs {
  long long E; int n_atoms, n_local, n_graphs, n_elements;
  const int64_t* edge_index;  // [2][E]
  const int* species; const int* graph_ptr;
  // outputs
  int* e_src; int* e_dst; int* e_orig;  // target-sorted
  int* rowptr_dst;            // [n_local+1]
  // split_rows: row_ids lists the owned targets none of whose sources is a ghost, then the others (each part in
  // ascending order); row_split[1] is the length of the first part
  int split_rows;
  int* row_ids;               // [n_local] or nullptr
  int* row_split;             // [2]
  int* perm_src; int* rowptr_src;       // [E], [n_atoms+1]
  int* atom_graph;            // [n_atoms]
  int* species_perm; int* species_ptr;  // [n_local], [n_elements+1]
  int* tile_ptr;              // [4][n_elements+1] for q = 1,3,5,7: 64-row tiles per species
  int* tc_tile_ptr;           // [4][n_elements+1]: (128 / q)-atom tiles per species
  void* temp; size_t temp_bytes;
};
size_t graph_prep_temp_bytes(long long E, int n_atoms);
cudaError_t launch_graph_prep(const GraphPrepArgs& a, cudaStream_t s);
// Edge chunks for systems whose per-edge tensors do not fit: chunk c = target atoms [atom_ptr[c], atom_ptr[c+1]) with
// atom_ptr[c] = first atom whose edge offset reaches c * target_edges; edge_ptr[c] = rowptr_dst[atom_ptr[c]].
cudaError_t launch_chunk_bounds(const int* rowptr_dst, int n_local, long long target_edges, int n_chunks, int* atom_ptr,
                                int* edge_ptr, cudaStream_t s);
// keys[k], perm[k]: edges sorted by (chunk, source atom); key = chunk * n_atoms + source.  temp as for launch_graph_prep.
cudaError_t launch_chunk_src_sort(const int* e_src, long long E, int n_atoms, const int* edge_ptr, int n_chunks, int* keys,
                                  int* perm, void* temp, size_t temp_bytes, cudaStream_t s);

}  // namespace tace

namespace tace {
// FP32-accurate GEMM on tcgen05 tensor cores (tc_gemm.cu): C[M,N] = A[M,K] @ B[N,K]^T with B given
// as its TF32 high part and residual.  `error_flag` (device int) receives a non-zero code if a
// bounded wait inside the kernel expired.
// Batched form for the per-rank linears: up to four problems per launch, rows = (atom, component) pairs
// addressed as base + atom * atom_stride + component * comp_stride (elements), K and N contiguous.
// ---- TECE edge block (tece_kernels.cu; tace/models/_e3nn/archive/oam_2026_07_05.py:547-823) --------------------
enum TeceStage {
  TECE_WIGNER, TECE_ROTATE_IN, TECE_LOGIT, TECE_SOFTMAX, TECE_MIX, TECE_ROTATE_OUT,
  TECE_ROTATE_OUT_BWD, TECE_ALPHA_BWD, TECE_SOFTMAX_BWD, TECE_LOGIT_BWD, TECE_EDGE_SCALAR_BWD, TECE_MIX_BWD,
  TECE_ROTATE_IN_BWD, TECE_TARGET_SUM, TECE_WIGNER_GRAD, TECE_WIGNER_BWD
};
// One argument block for every kernel of the edge block (layouts are described at the top of tece_kernels.cu).
template <typename T>
struct TeceArgs {
  long long E; int n_local, C, Ca, L, mmax, H, NR, NC, G, n_paths, gate_m0, act, accumulate_gvec;
  int row_l[16], row_m[16], row_comp[16]; T row_scale[16];          // order-major rows: rank, signed order, weight component, inverse rescale
  int p_m1[12], p_m2[12], p_m3[12], p_sum[12]; T p_scale[12];        // cluster-expansion paths
  RadialParams<T> rp;
  const T* vec; const T* dlen; const T* env;                         // env == nullptr: no cutoff factor (apply_cutoff = True)
  const int* e_src; const int* e_dst; const int* rowptr;
  const T* x; T* W; T* Wg; T* Ks; T* Qt; T* Mw; T* Kp; T* Qp; T* logit; T* alpha;
  const T* temp; const T* rproj_w; const T* rproj_b;                 // per-head scale * temperature; radial projection [8][2H], [2H]
  T* up; T* glu; T* coefZ; T* U; T* down; T* M;
  const T* gM; T* gdown; T* galpha; T* glogit; T* gcut; T* gproj; T* proj; T* gQp; T* gKp; T* gKs; T* gQt; T* gMw;
  const T* gU; T* gup; T* gglu; T* gcoefZ; T* gWg; T* gvec; T* dxe; T* dxt; T* gx; T* ddlen_extra;
};
template <typename T> cudaError_t launch_tece(const TeceArgs<T>& a, int stage, cudaStream_t s);

struct TcLinearProblem {
  const float* A; long long a_atom_stride, a_comp_stride;
  int q;                 // components per atom (2l+1), <= 128
  long long n_atoms;
  int K, N;
  const float* Bhi; const float* Blo;  // [N][K]
  float* C; long long c_s1, c_s2;
  const float* bias;     // [N] or nullptr
  // per-species form: atoms of A are sorted by species; group g owns atoms [group_ptr[g], group_ptr[g+1]) and tiles
  // [tile_ptr[g], tile_ptr[g+1]) of 128 / q atoms (device arrays); weights / bias of group g sit b_group_stride /
  // bias_group_stride elements apart; rows of C go to atom_map[sorted atom] (nullptr: same order as A)
  int n_groups;          // 0: a single group (plain linear)
  const int* group_ptr; const int* tile_ptr; const int* atom_map;
  long long b_group_stride, bias_group_stride;
  int accumulate;        // C += instead of C =
  int b_tiled;           // Bhi / Blo are stored K-tile-major, [groups][K/32][N][32] (b_group_stride must be N*K)
};
bool tc_linear_supported(int N, int K);
cudaError_t launch_tc_linear(const TcLinearProblem* probs, int n_problems, int* error_flag, cudaStream_t s);
cudaError_t launch_tc_gemm(const float* A, long long lda, const float* Bhi, const float* Blo, float* C, long long ldc, int M,
                           int N, int K, int* error_flag, cudaStream_t s, const float* bias = nullptr);
}  // namespace tace
