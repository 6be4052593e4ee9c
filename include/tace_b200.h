/*
 * C ABI of libtace_b200.so: TACE energy / conservative force / virial evaluation and the
 * cell-list neighbour list as hand-written CUDA kernels for sm_100a.
 *
 * The reference (xvzemin/tace) is pure Python: there is no foreign-function interface to
 * mirror, so each entry point cites the Python interface it stands behind (paths relative
 * to the reference project root).  Conventions:
 *   - plain pointers and sizes only; every array argument is DEVICE memory owned by the
 *     caller unless a comment says "host"; the library never frees caller memory;
 *   - all work is enqueued on the given stream, nothing synchronises except where stated;
 *   - every function returns an int status (0 = ok, negative = error, see
 *     tace_status_string); no C++ exception crosses the boundary, nothing traps or aborts;
 *   - a TaceModel is not re-entrant (one call at a time); distinct models are independent;
 *   - there is no CPU fallback: without a CUDA device tace_create fails.
 */
#ifndef TACE_B200_H
#define TACE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct TaceModel TaceModel;
typedef void* tace_stream_t; /* a cudaStream_t */

enum {
  TACE_OK = 0,
  TACE_ERR_INVALID_ARGUMENT = -1,
  TACE_ERR_UNSUPPORTED_CONFIG = -2,
  TACE_ERR_CAPACITY = -3,
  TACE_ERR_CUDA = -4,
  TACE_ERR_NO_DEVICE = -5,
  TACE_ERR_UNKNOWN_WEIGHT = -6,
  TACE_ERR_WEIGHTS_MISSING = -7
};

enum { TACE_F32 = 0, TACE_F64 = 1 };

/* Hyper-parameters of the model body.  Stands behind the constructor
 * tace.models.e3nnTACE(**cfg) (tace/models/_e3nn/tace.py:29-62) after
 * check_model_config (tace/models/_e3nn/default.py:231-316), for the options this path
 * supports: cgtp interaction + cgtp product basis, natural parity, Lmax == lmax. */
typedef struct {
  int dtype;          /* TACE_F32 or TACE_F64 */
  int L;              /* rank of the angular features and the atomic basis (the reference's lmax), 1..3 */
  int num_layers;     /* >= 1 */
  int num_channel;    /* multiple of 32, <= 256 */
  int num_elements;   /* length of the sorted atomic-number list */
  int correlation;    /* product-basis correlation order: 1, 2 or 3 */
  int num_bessel;     /* must be 8 */
  int mlp_hidden;     /* must be 64 (three hidden layers) */
  int envelope_p;     /* polynomial cutoff exponent (default 5) */
  int readout_hidden; /* width of the energy read-out hidden layer (default 16, <= 64) */
  double cutoff;
  double avg_num_neighbors;
  int Lnode;          /* rank of the node features between layers (the reference's Lmax), 1..L; 0 means "same as L".
                         Lnode < L needs correlation >= 2 (tace/models/_e3nn/base.py:113-360) */
  int use_alllayer;   /* readout_emlp.use_alllayer: every layer below the last adds a linear read-out of its scalar
                         channels (tace/models/_e3nn/readout.py:192-221); weights "ro.lin<t>" */
  int gate_m0_off;    /* 0: atomic_basis.gate_m0 = True (every rank, l = 0 included, scaled by a sigmoid gate; the
                         reference default); 1: gate_m0 = False (scalars through SiLU, ranks >= 1 gated; nonlinear.py:43-70) */
  int mlp_layers;     /* hidden layers of the radial MLP (radial_basis.hidden, all 64 wide): 1..3; 0 means 3 */
  int mlp_bias;       /* radial_basis.bias: every layer of the radial MLP has a bias ("t<i>.b0".."b3") */
  int env_after_mlp;  /* radial_basis.apply_cutoff = False: the polynomial envelope multiplies the output of the radial MLP
                         instead of the radial basis (tace/models/radial.py:974-993, _e3nn/inter.py:174-183) */
  int edge_update_element2; /* edge_update.type = element2: species embeddings of target and source are appended to the
                         radial features (tace/models/_e3nn/edge.py:190-257); folded into the tables "t<i>.tdst" / "tsrc".
                         As in the reference, edge features wider than the radial basis also put a LayerNorm before every
                         hidden activation of the radial MLP (tace/models/_e3nn/base.py:183-185, tace/models/mlp.py:172-176):
                         affine weights "t<i>.ln<j>g" / "t<i>.ln<j>b", [64] each */
  int num_fidelities; /* entries of `statistics` (multi-head read-out, tace/models/_e3nn/readout.py:18-33,72-84): the
                         read-out weights, species scales and isolated-atom energies carry a leading fidelity axis and
                         TaceBatch.fidelity picks the head per graph; 0 means 1 */
  int zbl;            /* short_range.zbl.enable (tace/models/radial.py:788-874, _e3nn/tace.py:387-408): 0 off; 1 pair
                         repulsion added to the read-out before the species scale (scale_shift.scale_zbl = True);
                         2 added after it.  Tables "zbl.z", "zbl.rcov" [num_elements] (atomic number, covalent radius)
                         and "zbl.par" = {0.529 * a_prefactor, a_exp}; the envelope power is envelope_p */
  int scatter_norm_density; /* atomic_basis.scatter_norm (tace/models/_e3nn/inter.py:102-110,249-260, base.py:240-249):
                         0 messages / avg_num_neighbors (folded into the packed linear_down weights); 1 "density": messages
                         / (beta * sum over incoming edges of tanh(MLP(radial)^2) [* envelope when env_after_mlp] + alpha);
                         2 "no_cutoff_density": the same without the envelope factor.  Weights "t<i>.dA0" [8][64], "dw1" [64],
                         "dab" = {alpha, beta} (+ "db0" [64], "db1" [1] with mlp_bias); not with edge_update_element2 */
  int resnet_identity; /* resnet.linear_type = identity (tace/models/_e3nn/residual.py:145-250): the skip connection of layers
                         above the first copies the ranks the layer output keeps instead of a per-species linear; no
                         "t<i>.res.*" weights.  (linear_type = agnostic needs no flag: the host repeats the one matrix for
                         every species, as it does for product_basis.agnostic) */
  int product_bilinear; /* product_basis.nonlinear = silu_bilineargate (tace/models/_e3nn/prod.py:58,87-155,183-247; correlation
                         2 only): the product's linear_up maps A to two factors x, y and to one SiLU gate per (path, channel);
                         the second-order basis is gate * (x (x) [y, 1]) with separate factors (no symmetry) and the
                         first-order coefficients act on x.  Weights "t<i>.pu.l<l>" [C][2C], "t<i>.pg" [C][paths*C], biases
                         "t<i>.pu.b" [2C], "t<i>.pg.b" [paths*C] */
  /* TECE edge block, atomic_basis.type = uv_so2 (tace/models/_e3nn/inter.py:440-519, _e3nn/archive/oam_2026_07_05.py:547-823):
     bit t of tece_layers makes interaction t (not the first; Lnode == L; whole-batch evaluation only) rotate the features of
     both ends of every edge into the edge frame, mix the orders |m| <= mmax (<= 2) with SO(2) linears, a gate and an edge
     cluster expansion of width edge_ace_hidden (0: num_channel), and weight the messages with num_head attention heads
     normalised over the incoming edges.  edge_act: 0 so2_sigmoid_gate, 1 so2_silu_gate.  Weights "t<i>.so2.<key|query|up|
     glu|coefs|down>.m<m>" ([K][N], transposed copies "...T.m<m>"), biases "t<i>.so2.<name>.b", "t<i>.att.temp" [heads]
     (attention scale * temperature), "t<i>.att.rw" [8][2 heads], "t<i>.att.rb" [2 heads]; the radial MLP of such a layer
     emits [rows per order][2 num_channel] weights */
  int tece_layers, mmax, num_head, edge_ace_hidden, edge_act;
  /* Tabulated radial weights (no reference counterpart; the reference evaluates the radial MLP for every edge,
     tace/models/_e3nn/inter.py:166-183).  With the identity edge update the MLP's output is a function of the edge
     length alone, so it can be read from a table: radial_table = K > 0 makes tace_forward interpolate the path weights
     of every interaction from "t<i>.rtab" [K][paths * num_channel][4] = (W, h dW/dd) at d = k h and at d = (k + 1) h,
     h = cutoff / K (cubic Hermite on interval k), inside the tensor-product kernels; no per-edge weight or hidden activation is
     stored and the radial MLP is never launched.  TACE_F32 models only, not with edge_update_element2 or tece_layers.
     0: the radial MLP runs per edge. */
  int radial_table;
} TaceConfig;

/* One batch of structures on the device.  Stands behind the `data` dictionary consumed by
 * TensorModel.forward (tace/models/adapter.py:32-41, 278-384).  Reals are in the model
 * dtype.  In graph mode `positions`, `lattice`, `edge_shifts` are given and edge vectors are
 * r[target] - r[source] + shift @ lattice[graph]; in edge-vector mode (the LAMMPS ML-IAP
 * path, tace/interface/lammps/mliap.py:117-136) `edge_vector` is given instead, atoms
 * [n_local, n_atoms) are ghosts that only act as message sources, and forces are returned
 * per edge. */
typedef struct {
  int64_t n_atoms;           /* local + ghost atoms */
  int64_t n_local;           /* atoms that receive messages and own an energy */
  int64_t n_edges;
  int32_t n_graphs;
  const void* positions;     /* [n_atoms,3] or NULL */
  const void* lattice;       /* [n_graphs,3,3] row vectors, or NULL */
  const int32_t* species;    /* [n_atoms] index into the model's element list */
  const int32_t* graph_ptr;  /* [n_graphs+1] first atom of each graph (atoms sorted by graph) */
  const int64_t* edge_index; /* [2,n_edges]: row 0 = source, row 1 = target (any order) */
  const void* edge_shifts;   /* [n_edges,3] or NULL */
  const void* edge_vector;   /* [n_edges,3] or NULL */
  const int32_t* fidelity;   /* [n_graphs] head of each graph (data["fidelity_idx"], tace/models/adapter.py:280-284),
                                or NULL for head 0 */
} TaceBatch;

/* Outputs, any of which may be NULL to skip it.  Stands behind the dictionary returned by
 * TensorModel.forward (tace/models/adapter.py:162-174, tace/models/_e3nn/tace.py:764-786):
 * forces = -dE/dr, virials = -dE/d(strain), stress = -virials/|det lattice|,
 * edge_forces = +dE/d(edge_vector). */
typedef struct {
  void* energy;      /* [n_graphs] */
  void* node_energy; /* [n_local] */
  void* forces;      /* [n_atoms,3] */
  void* virials;     /* [n_graphs,3,3] */
  void* stress;      /* [n_graphs,3,3] */
  void* edge_forces; /* [n_edges,3], in the caller's edge order */
} TaceOutputs;

const char* tace_status_string(int status);

/* tace.models.e3nnTACE(**cfg): validates the configuration, selects the current CUDA device
 * (must be compute capability 10.x) and allocates the weight arena. */
int tace_create(const TaceConfig* cfg, TaceModel** out);
void tace_destroy(TaceModel* model);

/* Weight arena.  Stands behind load_state_dict / the `.pt` checkpoint contract
 * (tace/lightning/lit_model.py:587-609,664-677): the host side repacks the reference's
 * parameters (normalisation constants folded in) into the named arrays listed here and
 * uploads each one (HOST pointer, model dtype).  tace_forward refuses to run until every
 * array has been set. */
int tace_weight_count(const TaceModel* model);
int tace_weight_info(const TaceModel* model, int index, const char** name, int64_t* numel);
int tace_set_weight(TaceModel* model, const char* name, const void* host_data, int64_t numel);

/* Bytes of device scratch tace_forward needs for a batch of this size. */
int tace_workspace_bytes(const TaceModel* model, int64_t n_atoms, int64_t n_local, int64_t n_edges,
                         int32_t n_graphs, size_t* bytes);

/* TensorModel.forward(data) (tace/models/adapter.py:32-41): energy, then the hand-written
 * backward pass for forces / virials / stress / edge forces (replaces the autograd call at
 * tace/models/adapter.py:95-104).  `workspace` is device memory of at least
 * tace_workspace_bytes bytes, 256-byte aligned. */
int tace_forward(TaceModel* model, const TaceBatch* batch, const TaceOutputs* out, void* workspace,
                 size_t workspace_bytes, tace_stream_t stream);

/* CUDA-graph replay of tace_forward (no reference counterpart; the reference relies on torch.compile /
 * AOT-Inductor for launch overhead, tace/compile/aot.py).  Enabled by default: the second tace_forward call
 * with the same n_atoms, n_local, n_edges, n_graphs, requested outputs and workspace is captured into a
 * CUDA graph; later calls copy the inputs into a staging area at the end of the workspace, launch the graph
 * on `stream` and copy the results out, so input and output pointers may differ from call to call.  Calls
 * with an exchange callback, with profiling enabled, or with new sizes run launch by launch.
 * tace_set_graph_mode(model, 0) switches replay off and frees the captured graphs;
 * tace_graph_replays returns how many calls were served by a graph launch. */
int tace_set_graph_mode(TaceModel* model, int enable);

/* Edge chunking (no reference counterpart: the reference materialises every per-edge tensor, which bounds the
 * system size by memory, tace/models/_e3nn/inter.py:185-285).  A batch with more than `max_edges` edges
 * (default 2^21, minimum 1024) is evaluated in chunks of target atoms holding about `max_edges` edges each; per-edge
 * activations, path weights and source gradients exist for one chunk at a time and are recomputed in the backward
 * pass.  tace_workspace_bytes reflects the setting, so call it after changing the limit.  A chunk always ends at an
 * atom boundary; an atom with more than 8192 neighbours makes tace_forward return a capacity error.  Chunked
 * passes read the chunk table back to the host once (one stream synchronisation per call). */
int tace_set_chunk_edges(TaceModel* model, int64_t max_edges);
int64_t tace_graph_replays(const TaceModel* model);

/* Ghost-row exchange for edge-vector mode with n_local < n_atoms and more than one layer.  Stands
 * behind lmp_data.forward_exchange / reverse_exchange as used by GhostExchange
 * (tace/models/lammps.py:82-129): before every layer after the first, tace_forward synchronises its
 * stream and calls fn(user, 0, in, out, n_atoms, vec_len): `in` holds the per-atom source features
 * [n_atoms, vec_len] (model dtype, device memory) with ghost rows zero, and the callback must fill
 * `out` with the same rows where every ghost row is a copy of its owner's row.  In the backward pass it
 * calls fn(user, 1, in, out, n_atoms, vec_len) with the gradient rows; the callback must write to `out`
 * the local rows plus the sum of the rows of their ghosts.  Both buffers belong to the workspace; the
 * callback must finish its device work (or order it on the stream of tace_forward) before returning.
 * Return 0 on success. */
typedef int (*tace_exchange_fn)(void* user, int reverse, const void* in, void* out, int64_t n_rows, int32_t vec_len);
int tace_set_exchange(TaceModel* model, tace_exchange_fn fn, void* user);
/* host_sync = 1 (default): tace_forward synchronises its stream before every callback, as a caller whose exchange runs on
 * another stream or on the host needs (LAMMPS' ML-IAP exchange, tace/models/lammps.py:82-102).  host_sync = 0: the callback
 * enqueues all of its device work on the stream of tace_forward (packing kernels, NCCL send / receive ordered on that
 * stream); tace_forward then calls it without synchronising and the host runs ahead of the GPU. */
int tace_set_exchange_sync(TaceModel* model, int host_sync);
/* Overlap of the exchange with the evaluation (needs host_sync = 0).  `stream` is a second stream of the same device on
 * which the callback enqueues all of its work (NULL, the default: none).  tace_forward makes that stream wait for the
 * rows the callback reads, calls the callback, and meanwhile goes on with the part of the layer that needs no ghost row:
 * the messages of the atoms none of whose neighbours is a ghost (forward), and, in the backward pass, the atoms with ghost
 * neighbours first, so that the gradient rows of the ghosts travel while the other atoms are processed.  It waits for the
 * exchange stream only where the exchanged rows are first read.  The reference has no counterpart: it calls
 * lmp_data.forward_exchange / reverse_exchange synchronously between two layers (tace/models/lammps.py:82-129).  Every
 * message sum keeps its order, so energies are bit-identical to those without a stream; gradient rows of atoms with several
 * ghost copies add the arrivals before the caller's own sum, so forces agree to rounding. */
int tace_set_exchange_stream(TaceModel* model, tace_stream_t stream);

/* Instrumentation (no counterpart in the reference, which has no tracing on this path):
 * tace_launch_count returns the number of this library's kernels enqueued by tace_forward so far
 * (CUB radix-sort launches are not counted).  With profiling enabled, tace_forward records a
 * CUDA event on its stream at every phase boundary; tace_profile_read synchronises on the events
 * of phase `index` of the last call and returns its name and device time in milliseconds. */
int64_t tace_launch_count(const TaceModel* model);
int tace_profile_enable(TaceModel* model, int enable);
int tace_profile_count(const TaceModel* model);
int tace_profile_read(TaceModel* model, int index, const char** name, float* ms);

/* Dense fp32 GEMM on the tcgen05 tensor cores with 3xTF32 operand splitting:
 * C[M,N] = A[M,K] @ B[N,K]^T, A row-major with leading dimension lda, B given K-major as its TF32 high
 * part B_hi and residual B_lo = B - B_hi, C row-major with leading dimension ldc.  K must be a multiple
 * of 32, N of 64, lda and ldc of 4, all pointers 16-byte aligned.  Stands behind the reference's
 * mlpLinear (torch.mm, tace/models/linear.py:267-276); tace_forward uses it for the last radial-MLP
 * layer of fp32 models.  `error_flag` is a device int that must be zero on entry; it receives a
 * non-zero code if a bounded wait inside the kernel expired (results are then undefined). */
int tace_tc_gemm_f32(const float* A, int64_t lda, const float* B_hi, const float* B_lo, float* C, int64_t ldc, int32_t M,
                     int32_t N, int32_t K, int32_t* error_flag, tace_stream_t stream);
/* Test mode of that kernel's bounded waits: every wait gives up after `spin_limit` polls (0: the normal 2^22), and every
 * load barrier expects `extra_expected_bytes` more than its loads deliver (0: normal), so that with a non-zero value it
 * never completes.  With both set, the next tace_tc_gemm_f32 records the code of the wait that ran out in `error_flag`
 * (1 ring slot free, 2 operands ready, 3 load landed, 4 accumulator free, 5 accumulator full), waits for the loads it has
 * issued, frees its tensor memory and returns without a result; no fault is involved.  Process-wide; reset with (0, 0). */
int tace_tc_gemm_set_test_mode(uint32_t spin_limit, uint32_t extra_expected_bytes);

/* Reads (and clears) the model's device-side error word: 0 = none; non-zero = a bounded wait in a
 * kernel launched by tace_forward expired.  Synchronises the device. */
int tace_device_error(TaceModel* model, int32_t* code);

/* Debug taps used by the parity tests: copies a named intermediate of the last tace_forward
 * call ("M0", "A0", "h1", ...) into `dst` (device, model dtype, at most `numel` elements).
 * Returns the number of elements copied or a negative status. */
int64_t tace_debug_read(TaceModel* model, const char* name, void* dst, int64_t numel, tace_stream_t stream);

/* Cell-list neighbour list for a batch of periodic structures.  Stands behind
 * get_neighborhood (tace/dataset/neighbour_list.py:195-298, matscipy "ijS" semantics): full
 * list, D = r_j - r_i + S @ cell, strict |D| < cutoff evaluated in fp64, self pairs kept
 * unless S = 0, no shifts along non-periodic axes.  Edges come out grouped by target atom.
 * Two calls: tace_nl_count fills `counts[n_atoms]` (neighbours per target atom); the caller
 * sizes the outputs; tace_nl_fill writes edge_index [2,n_edges] (row 0 = source, row 1 =
 * target) and integer shifts [n_edges,3].
 * positions/lattice are fp64, pbc is [n_graphs,3] bytes. `row_ptr` is int64 [n_atoms+1]
 * (exclusive prefix sum of counts, computed by the caller).  Both calls take their temporaries
 * (bins, sort keys, cell starts, sort scratch) from `workspace`, device memory of the caller of at
 * least tace_nl_workspace_bytes(n_atoms, n_graphs) bytes; they allocate nothing and do not
 * synchronise. */
int tace_nl_workspace_bytes(int64_t n_atoms, int32_t n_graphs, size_t* bytes);
int tace_nl_count(const double* positions, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr,
                  int32_t n_graphs, int64_t n_atoms, double cutoff, int32_t* counts, void* workspace, size_t workspace_bytes,
                  tace_stream_t stream);
int tace_nl_fill(const double* positions, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr,
                 int32_t n_graphs, int64_t n_atoms, double cutoff, const int64_t* row_ptr, int64_t n_edges,
                 int64_t* edge_index, int32_t* edge_shifts, void* workspace, size_t workspace_bytes, tace_stream_t stream);

/* Neighbour list in one call that allocates nothing.  No counterpart in the reference.
 *
 * For hosts that must not allocate device memory while they run: an MD engine that has handed all of
 * the GPU's memory to its own pool (LAMMPS/Kokkos style) so a cudaMalloc inside a plugin can fail or
 * fragment it, or a latency-sensitive loop that cannot afford the device-wide synchronisation a
 * cudaMalloc/cudaFree pair implies.  tace_nl_count / tace_nl_fill need a workspace sized by the caller and a
 * host round trip for the edge count (the caller allocates the outputs between the two calls); this variant keeps its
 * temporaries (bins, sort keys, cell starts, sort workspace) in a fixed 2 MiB device array built into
 * the library (every GPU that loads the library holds those 2 MiB until the process exits), computes
 * the row pointers on the device and fills the caller's edge arrays directly.  It calls no cudaMalloc,
 * cudaFree or allocating library routine.
 *
 * Limits: n_atoms <= 16384 and n_graphs <= 1024, otherwise TACE_ERR_CAPACITY and nothing is launched.
 * Outputs (device memory of the caller): row_ptr int64 [n_atoms+1] (exclusive prefix sum of the
 * neighbour counts; row_ptr[n_atoms] is the number of edges found), edge_index int64 [2, max_edges]
 * (row stride max_edges; row 0 = source, row 1 = target), edge_shifts int32 [max_edges, 3].  Edges
 * beyond max_edges are not written: compare row_ptr[n_atoms] with max_edges after the stream has
 * finished.  Edge order and content are identical to tace_nl_count + tace_nl_fill.
 *
 * The first call on a device looks up the device address of the built-in array (with that device
 * current); make that first call before any stream capture.  All calls share the one array, so two
 * calls that overlap on the GPU (different streams, or different host threads) race; calls on one
 * stream are safe back to back, and every call overwrites all scratch it later reads, so nothing needs
 * clearing between calls. */
int tace_nl_build_noalloc(const double* positions, const double* lattice, const uint8_t* pbc, const int32_t* graph_ptr,
                          int32_t n_graphs, int64_t n_atoms, double cutoff, int64_t max_edges, int64_t* row_ptr,
                          int64_t* edge_index, int32_t* edge_shifts, tace_stream_t stream);

/* ---- molecular dynamics on the device (domain-decomposed driver) -------------------------------------
 * The reference ships no integrator: its MD examples run under LAMMPS (`fix nve`, docs lammps.rst) or
 * ASE, which call the model once per step through tace/interface/lammps/mliap.py:96-115 or
 * tace/interface/ase/calculator.py:128-178.  These entry points keep the rest of such a step on the GPU.
 * All pointers are device pointers; every call is asynchronous on `stream`.
 *
 * tace_md_kick_drift: v += kick * F * inv_mass (skipped when forces == NULL), then x += dt * v (skipped
 *   when positions == NULL).  positions / velocities fp64 [n_atoms,3]; forces [n_atoms,3] in force_dtype
 *   (TACE_F32 / TACE_F64); inv_mass fp64 [n_atoms].  Units are the caller's (kick carries dt/2 and the
 *   unit conversion).
 * tace_md_langevin: v_i <- c1 v_i + sqrt((1 - c1^2) * kt_scaled * inv_mass_i) * xi with xi standard normal: the exact
 *   Ornstein-Uhlenbeck update over one step, c1 = exp(-friction * dt); kt_scaled is k_B T in the caller's velocity
 *   units (mass * velocity^2).  xi is a pure function of (seed, step, ids[i] or i, component): the same trajectory for
 *   any distribution of the atoms over ranks.  (The reference runs thermostats through ASE or LAMMPS.)
 * tace_md_kinetic_energy: out[0] = sum_i 0.5 * mass_i * |v_i|^2 in a fixed summation order; scratch holds
 *   at least 1024 doubles.
 * tace_edge_vectors: out[e] = positions[target_e] - positions[source_e] evaluated in fp64 and rounded to
 *   `dtype` (edge_index int64 [2,n_edges], row 0 = source); the edge-vector input of tace_forward
 *   (tace/models/adapter.py:341-352 computes the same difference in the model dtype).
 * tace_edges_within: keep[e] = 1 where |positions[target_e] - positions[source_e]|^2 < cutoff^2, in fp64 with the
 *   neighbour-list kernel's operation order: filters a list built with cutoff + skin down to the edges a fresh list
 *   with `cutoff` would hold (LAMMPS keeps such a skin list, `neighbor 2.0 bin`, docs/source/guide/lammps.rst:125;
 *   the reference's ASE calculator rebuilds its list on every call, tace/interface/ase/calculator.py:132-152).
 * tace_edges_scan / tace_edges_compact: the filtered list itself.  tace_edges_scan writes, for every edge of the list,
 *   the number of kept edges before it (`position`, exclusive sum of `keep`; fewer than 2^31 edges) and the number kept
 *   (`total`, one device int64 the caller reads to size the outputs); scratch from the caller
 *   (tace_edges_scan_workspace_bytes).  tace_edges_compact then writes the kept edges in list order (out_index int64
 *   [2,n_kept], so a list sorted by target stays sorted) and their vectors (out_vec [n_kept,3] in `dtype`, the same
 *   fp64 difference as tace_edge_vectors).
 * tace_rows_gather: dst[r,:] = src[index[r],:] for r < n_rows (packs a halo message; elem_bytes 4 or 8).
 * tace_rows_scatter_add: dst[index[r],:] += src[r,:]; the indices of one call must be distinct (unpacks
 *   gradients returned by a neighbouring domain, tace/models/lammps.py:105-129); float / double rows. */
int tace_md_kick_drift(double* positions, double* velocities, const void* forces, int32_t force_dtype, const double* inv_mass,
                       int64_t n_atoms, double kick, double dt, tace_stream_t stream);
int tace_md_langevin(double* velocities, const double* inv_mass, const int64_t* ids, int64_t n_atoms, double c1,
                     double kt_scaled, uint64_t seed, uint64_t step, tace_stream_t stream);
int tace_md_kinetic_energy(const double* velocities, const double* mass, int64_t n_atoms, double* scratch, double* out,
                           tace_stream_t stream);
int tace_edge_vectors(const double* positions, const int64_t* edge_index, int64_t n_edges, void* out, int32_t dtype,
                      tace_stream_t stream);
int tace_edges_within(const double* positions, const int64_t* edge_index, int64_t n_edges, double cutoff, uint8_t* keep,
                      tace_stream_t stream);
int tace_edges_scan_workspace_bytes(int64_t n_edges, size_t* bytes);
int tace_edges_scan(const uint8_t* keep, int64_t n_edges, int32_t* position, int64_t* total, void* workspace,
                    size_t workspace_bytes, tace_stream_t stream);
int tace_edges_compact(const double* positions, const int64_t* edge_index, int64_t n_edges, const uint8_t* keep,
                       const int32_t* position, int64_t n_kept, int64_t* out_index, void* out_vec, int32_t dtype,
                       tace_stream_t stream);
int tace_rows_gather(const void* src, const int64_t* index, int64_t n_rows, int32_t row_len, int32_t elem_bytes, void* dst,
                     tace_stream_t stream);
int tace_rows_scatter_add(const void* src, const int64_t* index, int64_t n_rows, int32_t row_len, int32_t elem_bytes, void* dst,
                          tace_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TACE_B200_H */
