// Host-side engine behind the C ABI (include/tace_b200.h): model plan, weight arena,
// workspace layout and the forward / hand-written backward schedule of one
// energy + forces + virial evaluation.
//
// Schedule of one call (reference: TensorModel.forward, tace/models/adapter.py:32-41, over
// Representation.forward, tace/models/_e3nn/representation.py:302-429):
//   graph prep -> edge features + radial MLP hidden layers -> per layer:
//   [linear_up, last radial layer (GEMM), tensor-product message passing, linear_down,
//    gate, linear, product basis, per-species coefficient linears, linear (+ skip)]
//   -> read-out -> the same chain in reverse with transposed weights -> edge-vector gradients
//   -> forces / virials / stress.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <string>
#include <type_traits>
#include <vector>

#include "../../include/tace_b200.h"
#include "gemm.cuh"
#include "kernels.h"
#include "tp_gen.cuh"

namespace tace {

namespace {

struct TPMeta { int NP, NX, NM, NG; const int* k; const int* base; };
struct PBMeta { int NP, NB; const int* k; const int* base; };

// L: rank of the angular features and messages; Lin: rank of the source features (< 0: scalar source)
bool tp_meta(int L, int Lin, TPMeta& m) {
#define TPM(TAG) { m = {TPX_##TAG::NP, TPX_##TAG::NX, TPX_##TAG::NM, TPX_##TAG::NG, tp_##TAG##_k, tp_##TAG##_base}; return true; }
  if (L == 1 && Lin < 0) TPM(L1_S)
  if (L == 1 && Lin == 1) TPM(L1_F)
  if (L == 2 && Lin < 0) TPM(L2_S)
  if (L == 2 && Lin == 1) TPM(L2_N1)
  if (L == 2 && Lin == 2) TPM(L2_F)
  if (L == 3 && Lin < 0) TPM(L3_S)
  if (L == 3 && Lin == 1) TPM(L3_N1)
  if (L == 3 && Lin == 2) TPM(L3_N2)
  if (L == 3 && Lin == 3) TPM(L3_F)
#undef TPM
  return false;
}
// L: rank of A; Lout: highest output rank (< 0: scalar outputs only)
bool pb_meta(int L, int Lout, PBMeta& m) {
#define PBM(TAG) { m = {PB_##TAG::NP, PB_##TAG::NB, pb_##TAG##_k, pb_##TAG##_base}; return true; }
  if (L == 1 && Lout < 0) PBM(L1_T)
  if (L == 1 && Lout == 1) PBM(L1_A)
  if (L == 2 && Lout < 0) PBM(L2_T)
  if (L == 2 && Lout == 1) PBM(L2_N1)
  if (L == 2 && Lout == 2) PBM(L2_A)
  if (L == 3 && Lout < 0) PBM(L3_T)
  if (L == 3 && Lout == 1) PBM(L3_N1)
  if (L == 3 && Lout == 2) PBM(L3_N2)
  if (L == 3 && Lout == 3) PBM(L3_A)
#undef PBM
  return false;
}

// gated bilinear product (two different factors, the second extended by a block of ones)
bool pbl_meta(int L, int Lout, PBMeta& m) {
#define PBM(TAG) { m = {PBL_##TAG::NP, PBL_##TAG::NB, pbl_##TAG##_k, pbl_##TAG##_base}; return true; }
  if (L == 1 && Lout < 0) PBM(L1_T)
  if (L == 1 && Lout == 1) PBM(L1_A)
  if (L == 2 && Lout < 0) PBM(L2_T)
  if (L == 2 && Lout == 1) PBM(L2_N1)
  if (L == 2 && Lout == 2) PBM(L2_A)
  if (L == 3 && Lout < 0) PBM(L3_T)
  if (L == 3 && Lout == 1) PBM(L3_N1)
  if (L == 3 && Lout == 2) PBM(L3_N2)
  if (L == 3 && Lout == 3) PBM(L3_A)
#undef PBM
  return false;
}

// third-order basis (correlation 3): L = rank of A, Lout as above
bool pb3_meta(int L, int Lout, PBMeta& m) {
#define PBM(TAG) { m = {PB3_##TAG::NP, PB3_##TAG::NB, pb3_##TAG##_k, pb3_##TAG##_base}; return true; }
  if (L == 1 && Lout < 0) PBM(L1_T)
  if (L == 1 && Lout == 1) PBM(L1_A)
  if (L == 2 && Lout < 0) PBM(L2_T)
  if (L == 2 && Lout == 1) PBM(L2_N1)
  if (L == 2 && Lout == 2) PBM(L2_A)
  if (L == 3 && Lout < 0) PBM(L3_T)
  if (L == 3 && Lout == 1) PBM(L3_N1)
  if (L == 3 && Lout == 2) PBM(L3_N2)
  if (L == 3 && Lout == 3) PBM(L3_A)
#undef PBM
  return false;
}

struct WeightEntry {
  std::string name;
  long long numel;
  long long offset;  // elements into the arena
  bool set;
};

struct LayerPlan {
  bool scalar_src, last, has_res;
  bool tece = false;        // the interaction is the TECE edge block (atomic_basis.type = uv_so2) instead of the tensor product
  TPMeta tp;
  PBMeta pb;                // second-order product basis (all ranks <= L when a third order follows)
  PBMeta pb3;               // third-order product basis (correlation 3)
  int pb_lout;              // output-rank argument of the second-order kernels
  int Din;                  // components per atom of the layer input (1 or D)
  int Dout;                 // components per atom of the layer output (D or 1)
  std::vector<int> in_ls;   // ranks present in the input
  std::vector<int> out_ls;  // ranks present in the output
};

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// Bump allocator over the caller's workspace; in "measure" mode it only counts.
struct Arena {
  unsigned char* base = nullptr;
  size_t used = 0;
  template <typename U>
  U* take(size_t count) {
    U* p = base ? reinterpret_cast<U*>(base + used) : nullptr;
    used += align256(sizeof(U) * (count ? count : 1));
    return p;
  }
};

}  // namespace

struct ModelBase {
  TaceConfig cfg;
  virtual ~ModelBase() {
    if (ev_fork) cudaEventDestroy(ev_fork);
    if (ev_join) cudaEventDestroy(ev_join);
  }
  // Runs the exchange callback.  Without an exchange stream: on the stream of the pass (after a host synchronisation when
  // the callback asks for one).  With one: everything enqueued on `s` so far happens before the callback's work, which
  // runs on the exchange stream; the pass goes on with `s` and calls exchange_join before it touches the callback's output.
  bool exchange_on_side() const { return exchange_stream != nullptr && !exchange_sync; }
  int exchange_begin(int reverse, const void* in, void* out, long long n_rows, int row, cudaStream_t s) {
    const bool side = exchange_on_side();
    if (side) {
      if (!ev_fork && (cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming) != cudaSuccess ||
                       cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming) != cudaSuccess))
        return TACE_ERR_CUDA;
      if (cudaEventRecord(ev_fork, s) != cudaSuccess || cudaStreamWaitEvent(exchange_stream, ev_fork, 0) != cudaSuccess)
        return TACE_ERR_CUDA;
    } else if (exchange_sync && cudaStreamSynchronize(s) != cudaSuccess) {
      return TACE_ERR_CUDA;
    }
    if (exchange_fn(exchange_user, reverse, in, out, n_rows, row) != 0) return TACE_ERR_INVALID_ARGUMENT;
    if (side && cudaEventRecord(ev_join, exchange_stream) != cudaSuccess) return TACE_ERR_CUDA;
    return TACE_OK;
  }
  int exchange_join(cudaStream_t s) {
    if (exchange_on_side() && cudaStreamWaitEvent(s, ev_join, 0) != cudaSuccess) return TACE_ERR_CUDA;
    return TACE_OK;
  }
  virtual int weight_count() const = 0;
  virtual int weight_info(int i, const char** name, int64_t* numel) const = 0;
  virtual int set_weight(const char* name, const void* host, int64_t numel) = 0;
  virtual int workspace_bytes(int64_t n_atoms, int64_t n_local, int64_t n_edges, int32_t n_graphs, size_t* bytes) = 0;
  virtual int forward(const TaceBatch* b, const TaceOutputs* o, void* ws, size_t ws_bytes, cudaStream_t s) = 0;
  virtual int64_t debug_read(const char* name, void* dst, int64_t numel, cudaStream_t s) = 0;

  // kernel-launch counter and optional per-phase CUDA-event timing
  long long launches = 0;
  // Batches with more edges than this are evaluated in chunks of target atoms: the per-edge tensors (radial-MLP
  // activations, path weights, per-edge source gradients) then exist for one chunk at a time and the backward pass
  // recomputes them, so memory per edge drops from kilobytes to about two hundred bytes.
  long long max_chunk_edges = 1LL << 21;
  tace_exchange_fn exchange_fn = nullptr;  // ghost-row exchange between layers (edge-vector mode)
  void* exchange_user = nullptr;
  bool exchange_sync = true;                // synchronise the stream before every exchange callback (tace_set_exchange_sync)
  // Stream on which the exchange callback enqueues its work (tace_set_exchange_stream).  The pass then orders the callback
  // against its own stream with events and keeps computing what does not need the ghost rows while they travel.
  cudaStream_t exchange_stream = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  int* dev_error = nullptr;  // device word written by kernels whose bounded waits expire
  bool profile = false;
  std::vector<std::string> phase_names;
  std::vector<cudaEvent_t> phase_events;
  size_t phase_used = 0;
  void phase(const char* name, cudaStream_t s) {
    if (!profile) return;
    if (phase_used == phase_events.size()) {
      cudaEvent_t e;
      if (cudaEventCreate(&e) != cudaSuccess) return;
      phase_events.push_back(e);
      phase_names.push_back("");
    }
    phase_names[phase_used] = name;
    cudaEventRecord(phase_events[phase_used], s);
    ++phase_used;
  }
  int phase_count() const { return phase_used > 0 ? (int)phase_used - 1 : 0; }
  int phase_read(int i, const char** name, float* ms) {
    if (i < 0 || i >= phase_count()) return TACE_ERR_INVALID_ARGUMENT;
    if (cudaEventSynchronize(phase_events[i + 1]) != cudaSuccess) return TACE_ERR_CUDA;
    if (cudaEventElapsedTime(ms, phase_events[i], phase_events[i + 1]) != cudaSuccess) return TACE_ERR_CUDA;
    *name = phase_names[i].c_str();
    return TACE_OK;
  }
  void release_events() {
    for (auto e : phase_events) cudaEventDestroy(e);
    phase_events.clear();
  }

  // ---- CUDA-graph replay ------------------------------------------------------------------------
  // A forward pass is several hundred short launches whose arguments depend only on the batch
  // sizes and the workspace address.  The second call with the same sizes is captured into a CUDA
  // graph on a private stream; from then on inputs are copied into a staging area at the end of
  // the workspace, the graph is launched on the caller's stream, and results are copied out, so
  // the caller's input and output pointers may change freely between calls.
  struct GraphKey {
    int64_t n_atoms, n_local, n_edges;
    int32_t n_graphs, vec_mode;  // vec_mode bit 0: edge-vector input; bit 1: a fidelity array is given
    uint32_t out_mask;
    void* ws;
    size_t ws_bytes;
    bool operator==(const GraphKey& o) const {
      return n_atoms == o.n_atoms && n_local == o.n_local && n_edges == o.n_edges && n_graphs == o.n_graphs &&
             vec_mode == o.vec_mode && out_mask == o.out_mask && ws == o.ws && ws_bytes == o.ws_bytes;
    }
  };
  struct GraphEntry { GraphKey key; cudaGraphExec_t exec; long long launches; unsigned long long last_use; };
  static constexpr size_t kMaxGraphs = 4, kMaxSeen = 16;
  int graph_mode = 1;
  std::vector<GraphKey> seen, rejected;
  std::vector<GraphEntry> graphs;
  cudaStream_t capture_stream = nullptr;
  unsigned long long graph_clock = 0;
  long long graph_replays = 0;

  struct Stage {  // byte offsets (from the staging base) of the copies of every input and output
    size_t positions, lattice, species, graph_ptr, edge_index, edge_shifts, edge_vector, fidelity;
    size_t energy, node_energy, forces, virials, stress, edge_forces, total;
  };
  Stage stage_layout(int64_t N, int64_t NL, int64_t E, int32_t B) const {
    const size_t ts = cfg.dtype == TACE_F32 ? 4 : 8;
    Stage st;
    size_t off = 0;
    auto take = [&off](size_t bytes) { const size_t at = off; off += align256(bytes ? bytes : 1); return at; };
    st.positions = take(ts * 3 * N); st.lattice = take(ts * 9 * B); st.species = take(4 * (size_t)N);
    st.graph_ptr = take(4 * (size_t)(B + 1)); st.edge_index = take(16 * (size_t)E); st.edge_shifts = take(ts * 3 * E);
    st.edge_vector = take(ts * 3 * E); st.fidelity = take(4 * (size_t)B);
    st.energy = take(ts * B); st.node_energy = take(ts * NL); st.forces = take(ts * 3 * N); st.virials = take(ts * 9 * B);
    st.stress = take(ts * 9 * B); st.edge_forces = take(ts * 3 * E);
    st.total = off;
    return st;
  }
  void release_graphs() {
    for (auto& g : graphs) cudaGraphExecDestroy(g.exec);
    graphs.clear(); seen.clear(); rejected.clear();
    if (capture_stream) { cudaStreamDestroy(capture_stream); capture_stream = nullptr; }
  }

  int forward_entry(const TaceBatch* bt, const TaceOutputs* o, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (!bt || !o || !ws) return TACE_ERR_INVALID_ARGUMENT;
    const int64_t N = bt->n_atoms, NL = bt->n_local, E = bt->n_edges;
    const int32_t B = bt->n_graphs;
    if (!graph_mode || profile || exchange_fn || N <= 0 || E <= 0 || B <= 0 || NL < 0 || NL > N || E > max_chunk_edges)
      return forward(bt, o, ws, ws_bytes, s);
    const Stage st = stage_layout(N, NL, E, B);
    if (ws_bytes < st.total + 256) return forward(bt, o, ws, ws_bytes, s);
    const size_t body_bytes = (ws_bytes - st.total) & ~size_t(255);
    unsigned char* sb = static_cast<unsigned char*>(ws) + body_bytes;
    GraphKey key{N, NL, E, B, (bt->edge_vector ? 1 : 0) | (bt->fidelity ? 2 : 0), 0u, ws, ws_bytes};
    const bool vec_in = bt->edge_vector != nullptr;
    const void* outs[6] = {o->energy, o->node_energy, o->forces, o->virials, o->stress, o->edge_forces};
    for (int k = 0; k < 6; ++k) if (outs[k]) key.out_mask |= 1u << k;
    // inputs the pass reads (all must be present for the staged path)
    if (!bt->species || !bt->graph_ptr || !bt->edge_index) return forward(bt, o, ws, ws_bytes, s);
    if (!vec_in && (!bt->positions || !bt->lattice || !bt->edge_shifts)) return forward(bt, o, ws, ws_bytes, s);

    GraphEntry* hit = nullptr;
    for (auto& g : graphs) if (g.key == key) hit = &g;
    if (!hit) {
      for (const auto& r : rejected) if (r == key) return forward(bt, o, ws, ws_bytes, s);
      bool was_seen = false;
      for (const auto& k : seen) if (k == key) was_seen = true;
      if (!was_seen) {  // first call with these sizes: run it directly (also configures kernel attributes)
        if (seen.size() >= kMaxSeen) seen.erase(seen.begin());
        seen.push_back(key);
        return forward(bt, o, ws, ws_bytes, s);
      }
      // second call: capture a pass that works on the staged copies
      if (!capture_stream && cudaStreamCreateWithFlags(&capture_stream, cudaStreamNonBlocking) != cudaSuccess)
        return forward(bt, o, ws, ws_bytes, s);
      TaceBatch sbt = *bt;
      TaceOutputs so;
      const size_t ts = cfg.dtype == TACE_F32 ? 4 : 8;
      (void)ts;
      sbt.species = reinterpret_cast<const int32_t*>(sb + st.species);
      sbt.graph_ptr = reinterpret_cast<const int32_t*>(sb + st.graph_ptr);
      sbt.edge_index = reinterpret_cast<const int64_t*>(sb + st.edge_index);
      sbt.positions = vec_in ? nullptr : sb + st.positions;
      sbt.lattice = vec_in ? nullptr : sb + st.lattice;
      sbt.edge_shifts = vec_in ? nullptr : sb + st.edge_shifts;
      sbt.edge_vector = vec_in ? sb + st.edge_vector : nullptr;
      sbt.fidelity = bt->fidelity ? reinterpret_cast<const int32_t*>(sb + st.fidelity) : nullptr;
      so.energy = o->energy ? sb + st.energy : nullptr;
      so.node_energy = o->node_energy ? sb + st.node_energy : nullptr;
      so.forces = o->forces ? sb + st.forces : nullptr;
      so.virials = o->virials ? sb + st.virials : nullptr;
      so.stress = o->stress ? sb + st.stress : nullptr;
      so.edge_forces = o->edge_forces ? sb + st.edge_forces : nullptr;
      const long long before = launches;
      cudaGraph_t graph = nullptr;
      cudaGraphExec_t exec = nullptr;
      bool ok = cudaStreamBeginCapture(capture_stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
      if (ok) {
        const int status = forward(&sbt, &so, ws, body_bytes, capture_stream);
        const cudaError_t ce = cudaStreamEndCapture(capture_stream, &graph);
        ok = status == TACE_OK && ce == cudaSuccess && graph != nullptr;
      }
      const long long per_pass = launches - before;
      launches = before;
      if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
      if (graph) cudaGraphDestroy(graph);
      if (!ok) {
        cudaGetLastError();  // a failed capture leaves a sticky-free error behind; this sizes runs without a graph
        rejected.push_back(key);
        return forward(bt, o, ws, ws_bytes, s);
      }
      if (graphs.size() >= kMaxGraphs) {
        size_t oldest = 0;
        for (size_t k = 1; k < graphs.size(); ++k) if (graphs[k].last_use < graphs[oldest].last_use) oldest = k;
        cudaGraphExecDestroy(graphs[oldest].exec);
        graphs.erase(graphs.begin() + oldest);
      }
      graphs.push_back({key, exec, per_pass, 0});
      hit = &graphs.back();
    }
    hit->last_use = ++graph_clock;
    const size_t ts = cfg.dtype == TACE_F32 ? 4 : 8;
    auto copy = [s](void* dst, const void* src, size_t bytes) {
      return bytes == 0 || cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s) == cudaSuccess;
    };
    bool ok = copy(sb + st.species, bt->species, 4 * (size_t)N) && copy(sb + st.graph_ptr, bt->graph_ptr, 4 * (size_t)(B + 1)) &&
              copy(sb + st.edge_index, bt->edge_index, 16 * (size_t)E);
    if (bt->fidelity) ok = ok && copy(sb + st.fidelity, bt->fidelity, 4 * (size_t)B);
    if (vec_in) ok = ok && copy(sb + st.edge_vector, bt->edge_vector, ts * 3 * E);
    else ok = ok && copy(sb + st.positions, bt->positions, ts * 3 * N) && copy(sb + st.lattice, bt->lattice, ts * 9 * B) &&
              copy(sb + st.edge_shifts, bt->edge_shifts, ts * 3 * E);
    if (!ok || cudaGraphLaunch(hit->exec, s) != cudaSuccess) return TACE_ERR_CUDA;
    launches += hit->launches;
    ++graph_replays;
    ok = (!o->energy || copy(o->energy, sb + st.energy, ts * B)) && (!o->node_energy || copy(o->node_energy, sb + st.node_energy, ts * NL)) &&
         (!o->forces || copy(o->forces, sb + st.forces, ts * 3 * N)) && (!o->virials || copy(o->virials, sb + st.virials, ts * 9 * B)) &&
         (!o->stress || copy(o->stress, sb + st.stress, ts * 9 * B)) &&
         (!o->edge_forces || copy(o->edge_forces, sb + st.edge_forces, ts * 3 * E));
    return ok ? TACE_OK : TACE_ERR_CUDA;
  }
};

template <typename T>
struct Model : ModelBase {
  int L, Ln, D, C, NL_, n_el, H;
  int nh = 3;                 // hidden layers of the radial MLP (radial_basis.hidden)
  bool mlp_bias = false;      // radial_basis.bias
  bool env_after = false;     // radial_basis.apply_cutoff = False: envelope multiplies the MLP output
  bool element2 = false;      // edge_update.type = element2
  int n_fid = 1;              // read-out heads (entries of `statistics`)
  int zbl = 0;                // 0 off, 1 ZBL repulsion inside the species scale, 2 outside it
  int density = 0;            // atomic_basis.scatter_norm: 0 avg_num_neighbors, 1 density, 2 no_cutoff_density
  bool res_identity = false;  // resnet.linear_type = identity: the skip connection copies the matching ranks, no weights
  bool bilinear = false;      // product_basis.nonlinear = silu_bilineargate: gated product of two linear images of A
  // TECE edge block: layers (bit t), orders kept, heads, width of the cluster expansion, activation (0 sigmoid, 1 SiLU)
  int tece_mask = 0, mmax = 2, heads = 1, Ca = 0, edge_act = 0;
  int rt_K = 0;               // > 0: path weights interpolated from per-layer tables with rt_K intervals (TaceConfig.radial_table)
  int t_NR = 0, t_NC = 0, t_NF = 0, t_G = 0, t_np = 0, t_WN = 0;  // rows (order-major / per weight / full), gates, paths, coefficients
  int t_k[4] = {1, 1, 1, 1}, t_base[4] = {0, 1, 4, 9};            // message layout of a TECE layer: one block of C per rank
  int t_row_l[16], t_row_m[16], t_row_comp[16]; double t_row_scale[16];
  int t_p_m1[12], t_p_m2[12], t_p_m3[12], t_p_sum[12]; double t_p_scale[12];
  int m0 = 1;  // 1: every rank gated (gate_m0 = True); 0: e3nn Gate, scalars through SiLU (gate_m0 = False)
  std::vector<LayerPlan> layers;
  std::vector<WeightEntry> weights;
  T* arena = nullptr;
  long long arena_numel = 0;
  struct DebugBuf { std::string name; const void* ptr; long long numel; };
  std::vector<DebugBuf> debug;
  T host_bessel[kNumBessel + 1];  // host copies of the radial frequencies and prefactor

  ~Model() override {
    if (arena) cudaFree(arena);
    if (dev_error) cudaFree(dev_error);
    release_events();
  }
  static constexpr bool kTensorCore = sizeof(T) == 4;  // fp32 models run the radial GEMMs on tcgen05

  void add_weight(const std::string& name, long long numel) {
    weights.push_back({name, numel, arena_numel, false});
    arena_numel += (numel + 63) / 64 * 64;
  }
  // a channel-mixing matrix used by the tensor-core path also needs its TF32 high part and residual
  void add_linear_weight(const std::string& name, long long numel) {
    add_weight(name, numel);
    if (kTensorCore) { add_weight(name + "_hi", numel); add_weight(name + "_lo", numel); }
  }
  const T* w(const std::string& name) const {
    for (const auto& e : weights)
      if (e.name == name) return arena + e.offset;
    return nullptr;
  }

  int init(const TaceConfig& c) {
    cfg = c;
    L = c.L; D = (L + 1) * (L + 1); C = c.num_channel; NL_ = c.num_layers; n_el = c.num_elements; H = c.readout_hidden;
    m0 = c.gate_m0_off ? 0 : 1;
    nh = (c.mlp_layers > 0) ? c.mlp_layers : 3;  // hidden layers of the radial MLP
    if (nh < 1 || nh > 3) return TACE_ERR_UNSUPPORTED_CONFIG;
    mlp_bias = c.mlp_bias != 0; env_after = c.env_after_mlp != 0; element2 = c.edge_update_element2 != 0;
    n_fid = c.num_fidelities > 0 ? c.num_fidelities : 1;
    zbl = c.zbl;
    density = c.scatter_norm_density;
    res_identity = c.resnet_identity != 0;
    bilinear = c.product_bilinear != 0;
    tece_mask = c.tece_layers; mmax = c.mmax; heads = c.num_head > 0 ? c.num_head : 1;
    rt_K = c.radial_table;
    if (rt_K < 0 || (rt_K > 0 && (!std::is_same<T, float>::value || element2 || tece_mask || rt_K > (1 << 16))))
      return TACE_ERR_UNSUPPORTED_CONFIG;
    Ca = c.edge_ace_hidden > 0 ? c.edge_ace_hidden : c.num_channel; edge_act = c.edge_act;
    if (tece_mask) {
      // the block needs ranks above 0 on its input (not the first layer), node rank = edge rank, orders <= 2
      if ((tece_mask & 1) || (c.Lnode > 0 && c.Lnode != c.L) || mmax < 0 || mmax > 2 || mmax > c.L || heads > 16 || C % heads ||
          Ca % 4 || density || (edge_act != 0 && edge_act != 1))
        return TACE_ERR_UNSUPPORTED_CONFIG;
      const int n = L + 1;
      t_NR = 0; t_NC = 0;
      for (int m = 0; m <= mmax; ++m) {
        for (int sign = 1; sign >= (m ? -1 : 1); sign -= 2)
          for (int l = m; l <= L; ++l) {
            t_row_l[t_NR] = l; t_row_m[t_NR] = sign * m; t_row_comp[t_NR] = t_NC + (l - m);
            t_row_scale[t_NR] = l > mmax ? std::sqrt((2.0 * l + 1.0) / (2.0 * mmax + 1.0)) : 1.0;
            ++t_NR;
          }
        t_NC += L + 1 - m;
      }
      t_NF = n + 2 * n * mmax;
      t_G = n * (mmax + 1 - (m0 ? 0 : 1));
      // cluster-expansion paths, output order major (oam_2026_07_05.py:331-369 with m1 >= m2)
      t_np = 0;
      for (int m3 = 0; m3 <= mmax; ++m3) {
        const int first = t_np;
        for (int m1 = 0; m1 <= mmax; ++m1)
          for (int m2 = 0; m2 <= m1; ++m2) {
            const bool sum = (m1 + m2 == m3), diff = !sum && (m1 - m2 == m3);
            if (!sum && !diff) continue;
            t_p_m1[t_np] = m1; t_p_m2[t_np] = m2; t_p_m3[t_np] = m3; t_p_sum[t_np] = sum ? 1 : 0; ++t_np;
          }
        for (int q = first; q < t_np; ++q) t_p_scale[q] = 1.0 / std::sqrt((double)(t_np - first));
      }
      t_WN = t_np * n * Ca;
    }
    if (bilinear && c.correlation != 2) return TACE_ERR_UNSUPPORTED_CONFIG;
    if (zbl < 0 || zbl > 2 || density < 0 || density > 2 || (density && element2)) return TACE_ERR_UNSUPPORTED_CONFIG;
    Ln = (c.Lnode > 0) ? c.Lnode : L;  // node features between layers carry ranks 0..Ln; A, Y and the messages 0..L
    if (Ln > L || (Ln < L && c.correlation < 2)) return TACE_ERR_UNSUPPORTED_CONFIG;
    const int Dn = (Ln + 1) * (Ln + 1);
    layers.resize(NL_);
    for (int t = 0; t < NL_; ++t) {
      LayerPlan& p = layers[t];
      p.scalar_src = (t == 0);
      p.last = (t == NL_ - 1);
      p.has_res = (t > 0);
      const int lout = p.last ? -1 : Ln;
      p.pb_lout = (c.correlation == 3) ? L : lout;  // with a third order the second keeps every rank (prod.py:216-266)
      p.pb3 = PBMeta{0, 0, nullptr, nullptr};
      if (!tp_meta(L, p.scalar_src ? -1 : Ln, p.tp) || !(bilinear ? pbl_meta(L, p.pb_lout, p.pb) : pb_meta(L, p.pb_lout, p.pb)))
        return TACE_ERR_UNSUPPORTED_CONFIG;
      if (c.correlation == 3 && !pb3_meta(L, lout, p.pb3)) return TACE_ERR_UNSUPPORTED_CONFIG;
      p.tece = (tece_mask >> t) & 1;
      if (p.tece) p.tp = TPMeta{2 * t_NC, D, D, 0, t_k, t_base};  // radial weights [NC][2C]; messages one C-block per rank
      p.Din = p.scalar_src ? 1 : Dn;
      p.Dout = p.last ? 1 : Dn;
      p.in_ls.clear(); p.out_ls.clear();
      for (int l = 0; l <= (p.scalar_src ? 0 : Ln); ++l) p.in_ls.push_back(l);
      for (int l = 0; l <= (p.last ? 0 : Ln); ++l) p.out_ls.push_back(l);
    }
    add_weight("emb", (long long)n_el * C);
    add_weight("bessel", kNumBessel);
    add_weight("bessel_pref", 1);
    for (int t = 0; t < NL_; ++t) {
      const LayerPlan& p = layers[t];
      const std::string pre = "t" + std::to_string(t) + ".";
      for (int l : p.in_ls) { add_linear_weight(pre + "up.l" + std::to_string(l), (long long)C * C); add_linear_weight(pre + "upT.l" + std::to_string(l), (long long)C * C); }
      add_weight(pre + "up.b", C);
      if (rt_K) add_weight(pre + "rtab", (long long)rt_K * p.tp.NP * C * 4);
      add_weight(pre + "A0", kNumBessel * kHidden);
      if (nh >= 2) { add_linear_weight(pre + "A1", kHidden * kHidden); add_linear_weight(pre + "A1t", kHidden * kHidden); }
      if (nh >= 3) { add_linear_weight(pre + "A2", kHidden * kHidden); add_linear_weight(pre + "A2t", kHidden * kHidden); }
      if (mlp_bias) {
        add_weight(pre + "b0", kHidden);
        if (nh >= 2) add_weight(pre + "b1", kHidden);
        if (nh >= 3) add_weight(pre + "b2", kHidden);
        add_weight(pre + "b3", (long long)p.tp.NP * C);
      }
      if (p.tece) {
        for (int i = 0; i < 6; ++i) {
          const So2Shape sh = so2_shape(i);
          for (int m = 0; m <= sh.mm; ++m) {
            const long long numel = (long long)sh.n_in[m] * sh.c_in * sh.n_out[m] * sh.c_out;
            add_linear_weight(pre + "so2." + sh.name + ".m" + std::to_string(m), numel);
            add_linear_weight(pre + "so2." + sh.name + "T.m" + std::to_string(m), numel);
          }
          add_weight(pre + "so2." + sh.name + ".b", (long long)sh.n_out[0] * sh.c_out);
        }
        add_weight(pre + "att.temp", heads); add_weight(pre + "att.rw", (long long)kNumBessel * 2 * heads); add_weight(pre + "att.rb", 2 * heads);
      }
      if (density) {  // edge-density MLP 8 -> 64 -> 1 and the affine parameters {alpha, beta}
        add_weight(pre + "dA0", (long long)kNumBessel * kHidden); add_weight(pre + "dw1", kHidden); add_weight(pre + "dab", 2);
        if (mlp_bias) { add_weight(pre + "db0", kHidden); add_weight(pre + "db1", 1); }
      }
      if (element2) {
        add_weight(pre + "tdst", (long long)n_el * kHidden); add_weight(pre + "tsrc", (long long)n_el * kHidden);
        // edge features wider than the radial basis put a LayerNorm before every hidden activation of the radial MLP
        // (tace/models/_e3nn/base.py:183-185, tace/models/mlp.py:172-176): affine weights per hidden layer
        for (int j = 0; j < nh; ++j) {
          add_weight(pre + "ln" + std::to_string(j) + "g", kHidden); add_weight(pre + "ln" + std::to_string(j) + "b", kHidden);
        }
      }
      add_weight(pre + "W3", (long long)kHidden * p.tp.NP * C);
      add_weight(pre + "W3t", (long long)kHidden * p.tp.NP * C);
      if (kTensorCore) {  // TF32 high parts and residuals of both orientations
        add_weight(pre + "W3_hi", (long long)kHidden * p.tp.NP * C);
        add_weight(pre + "W3_lo", (long long)kHidden * p.tp.NP * C);
        add_weight(pre + "W3t_hi", (long long)kHidden * p.tp.NP * C);
        add_weight(pre + "W3t_lo", (long long)kHidden * p.tp.NP * C);
      }
      for (int l = 0; l <= L; ++l) {
        const long long outl = (l == 0) ? (long long)(L + 1 + m0) * C : C;
        add_linear_weight(pre + "down.l" + std::to_string(l), (long long)p.tp.k[l] * C * outl);
        add_linear_weight(pre + "downT.l" + std::to_string(l), (long long)p.tp.k[l] * C * outl);
        add_linear_weight(pre + "nl.l" + std::to_string(l), (long long)C * C);
        add_linear_weight(pre + "nlT.l" + std::to_string(l), (long long)C * C);
      }
      add_weight(pre + "down.b", (long long)(L + 1 + m0) * C);
      add_weight(pre + "nl.b", C);
      for (size_t i = 0; i < p.out_ls.size(); ++i) {
        const int l = p.out_ls[i];
        const std::string ls = std::to_string(l);
        add_linear_weight(pre + "c0.l" + ls, (long long)n_el * C * C);
        add_linear_weight(pre + "c0T.l" + ls, (long long)n_el * C * C);
        if (cfg.correlation >= 2) {
          add_linear_weight(pre + "c1.l" + ls, (long long)n_el * p.pb.k[i] * C * C);
          add_linear_weight(pre + "c1T.l" + ls, (long long)n_el * p.pb.k[i] * C * C);
        }
        if (cfg.correlation >= 3) {
          add_linear_weight(pre + "c2.l" + ls, (long long)n_el * p.pb3.k[i] * C * C);
          add_linear_weight(pre + "c2T.l" + ls, (long long)n_el * p.pb3.k[i] * C * C);
        }
        add_linear_weight(pre + "lin.l" + ls, (long long)C * C);
        add_linear_weight(pre + "linT.l" + ls, (long long)C * C);
        if (p.has_res && !res_identity) {
          add_linear_weight(pre + "res.l" + ls, (long long)n_el * C * C);
          add_linear_weight(pre + "resT.l" + ls, (long long)n_el * C * C);
        }
      }
      if (bilinear) {  // linear_up of the product: every rank to both factors, the scalars also to the gates
        for (int l = 0; l <= L; ++l) {
          add_linear_weight(pre + "pu.l" + std::to_string(l), (long long)C * 2 * C);
          add_linear_weight(pre + "puT.l" + std::to_string(l), (long long)C * 2 * C);
        }
        add_linear_weight(pre + "pg", (long long)C * p.pb.NP * C);
        add_linear_weight(pre + "pgT", (long long)C * p.pb.NP * C);
        add_weight(pre + "pu.b", 2 * C);
        add_weight(pre + "pg.b", (long long)p.pb.NP * C);
      }
      add_weight(pre + "c.b", (long long)n_el * C);
      add_weight(pre + "lin.b", C);
      if (p.has_res && !res_identity) add_weight(pre + "res.b", (long long)n_el * C);
    }
    add_weight("ro.W1", (long long)n_fid * C * H);
    add_weight("ro.W2", (long long)n_fid * H);
    if (c.use_alllayer)
      for (int t = 0; t + 1 < NL_; ++t) add_weight("ro.lin" + std::to_string(t), (long long)n_fid * C);
    add_weight("scale", (long long)n_fid * n_el);
    add_weight("e0", (long long)n_fid * n_el);
    if (zbl) { add_weight("zbl.z", n_el); add_weight("zbl.rcov", n_el); add_weight("zbl.par", 2); }
    if (cudaMalloc(&arena, sizeof(T) * (size_t)arena_numel) != cudaSuccess) return TACE_ERR_CUDA;
    if (cudaMemset(arena, 0, sizeof(T) * (size_t)arena_numel) != cudaSuccess) return TACE_ERR_CUDA;
    if (cudaMalloc(&dev_error, sizeof(int)) != cudaSuccess || cudaMemset(dev_error, 0, sizeof(int)) != cudaSuccess)
      return TACE_ERR_CUDA;
    return TACE_OK;
  }

  int weight_count() const override { return (int)weights.size(); }
  int weight_info(int i, const char** name, int64_t* numel) const override {
    if (i < 0 || i >= (int)weights.size()) return TACE_ERR_INVALID_ARGUMENT;
    if (name) *name = weights[i].name.c_str();
    if (numel) *numel = weights[i].numel;
    return TACE_OK;
  }
  int set_weight(const char* name, const void* host, int64_t numel) override {
    if (!name || !host) return TACE_ERR_INVALID_ARGUMENT;
    for (auto& e : weights) {
      if (e.name == name) {
        if (numel != e.numel) return TACE_ERR_INVALID_ARGUMENT;
        if (cudaMemcpy(arena + e.offset, host, sizeof(T) * (size_t)numel, cudaMemcpyHostToDevice) != cudaSuccess)
          return TACE_ERR_CUDA;
        if (e.name == "bessel") memcpy(host_bessel, host, sizeof(T) * kNumBessel);
        if (e.name == "bessel_pref") memcpy(host_bessel + kNumBessel, host, sizeof(T));
        e.set = true;
        return TACE_OK;
      }
    }
    return TACE_ERR_UNKNOWN_WEIGHT;
  }

  // ---- workspace ---------------------------------------------------------------------------
  static constexpr long long kChunkSlack = 8192;  // a chunk ends at an atom boundary: room for one atom's edges beyond the target
  struct LayerBufs {
    T *h_in, *x, *xx, *gxx, *W, *H3, *Z1, *Z2, *Z3, *Hact, *M, *Gt, *gGt, *a, *A, *B2, *out, *h_out;
    T *gh_out, *gout, *gA, *ga, *gx, *gh_in;
    T *As, *gAs, *gout_s, *hs;  // species-sorted copies used by the per-species linears
    T *B3, *gB2;                // third-order basis (reused for its gradient) and the gradient of the second-order one
    T *inv_density, *gdens;     // learned edge density: 1 / density_i and dE / d density_i
    T *XY, *gXY, *Zg, *gZg;     // gated bilinear product: both factors per (atom, component), gate pre-activations, gradients
    // TECE edge block (layouts at the top of tece_kernels.cu); gradients that may overwrite their forward buffer do
    T *tKs, *tQt, *tMw, *tKp, *tQp, *tlogit, *talpha, *tup, *tglu, *tcoef, *tU, *tdown;
    T *tgdown, *tgalpha, *tglogit, *tgcut, *tgproj, *tproj, *tgQp, *tgKp, *tgKs, *tgQt, *tdxt, *tddlen;
  };
  struct Bufs {
    int *row_ids, *row_split;  // owned targets without / with a ghost source (passes split around the exchange)
    int *e_src, *e_dst, *e_orig, *perm_src, *rowptr_dst, *rowptr_src, *atom_graph, *species_perm, *species_ptr, *tile_ptr, *tc_tile_ptr;
    int *chunk_atom_ptr, *chunk_edge_ptr, *keys_cs, *perm_cs;  // edge chunks; (chunk, source)-sorted edge list
    int n_chunks; long long chunk_rows;                        // rows held by the per-edge chunk buffers
    void* prep_temp; size_t prep_temp_bytes;
    T *energy_partial;  // slice sums of the per-graph energies (graph_energy_slices)
    T *vec, *Y, *dY, *g, *e_scaled, *atom_virial, *dxe, *dlen, *ddlen, *ro_factor, *env, *denv, *zbl_node;
    T *tWg, *tgWg, *tgvec;  // TECE: Wigner rows of every edge (shared by the layers), their gradient, dE/d(edge vector) through them
    std::vector<LayerBufs> lay;
  };

  size_t layout(Arena& ar, Bufs& b, long long N, long long NL, long long E, int B) {
    b.e_src = ar.take<int>(E); b.e_dst = ar.take<int>(E); b.e_orig = ar.take<int>(E); b.perm_src = ar.take<int>(E);
    b.rowptr_dst = ar.take<int>(NL + 1); b.rowptr_src = ar.take<int>(N + 1); b.atom_graph = ar.take<int>(N);
    b.row_ids = ar.take<int>(NL); b.row_split = ar.take<int>(2);
    b.species_perm = ar.take<int>(NL); b.species_ptr = ar.take<int>(n_el + 1); b.tile_ptr = ar.take<int>(4 * (n_el + 1));
    b.tc_tile_ptr = ar.take<int>(4 * (n_el + 1));
    b.prep_temp_bytes = graph_prep_temp_bytes(E, (int)N);
    b.prep_temp = ar.take<unsigned char>(b.prep_temp_bytes);
    b.vec = ar.take<T>(3 * E); b.Y = ar.take<T>((size_t)D * E); b.dY = ar.take<T>((size_t)D * E); b.g = ar.take<T>(3 * E);
    b.energy_partial = ar.take<T>((size_t)B * graph_energy_slices(NL, B));
    b.e_scaled = ar.take<T>(NL); b.atom_virial = ar.take<T>(9 * NL); b.ro_factor = ar.take<T>(NL); b.zbl_node = zbl ? ar.take<T>(NL) : nullptr;
    b.tWg = b.tgWg = b.tgvec = nullptr;
    if (tece_mask) { b.tWg = ar.take<T>((size_t)E * t_NR * D); b.tgWg = ar.take<T>((size_t)E * t_NR * D); b.tgvec = ar.take<T>(3 * (size_t)E); }
    b.dlen = ar.take<T>(E); b.ddlen = ar.take<T>(E);
    b.env = env_after ? ar.take<T>(E) : nullptr; b.denv = env_after ? ar.take<T>(E) : nullptr;
    const bool chunked = E > max_chunk_edges;
    b.n_chunks = chunked ? (int)((E + max_chunk_edges - 1) / max_chunk_edges) : 1;
    b.chunk_rows = chunked ? max_chunk_edges + kChunkSlack : E;
    const long long Ec = b.chunk_rows;
    b.chunk_atom_ptr = ar.take<int>(b.n_chunks + 1); b.chunk_edge_ptr = ar.take<int>(b.n_chunks + 1);
    b.keys_cs = chunked ? ar.take<int>(E) : nullptr; b.perm_cs = chunked ? ar.take<int>(E) : nullptr;
    b.dxe = NL_ > 1 ? ar.take<T>((size_t)Ec * D * C) : nullptr;  // per-edge gradient rows of the source features
    T* shared_edge[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    T* shared_W = nullptr;
    if (chunked && !rt_K) {  // one set of chunk-sized per-edge buffers serves every layer
      for (int k = 0; k < 5; ++k) shared_edge[k] = ar.take<T>((size_t)Ec * kHidden);
      int np_max = 0;
      for (const auto& p : layers) np_max = p.tp.NP > np_max ? p.tp.NP : np_max;
      shared_W = ar.take<T>((size_t)Ec * np_max * C);
    }
    b.lay.resize(NL_);
    T* prev_h = ar.take<T>((size_t)N * C);   // h_0: species embedding, scalar channels
    T* prev_gh = nullptr;
    for (int t = 0; t < NL_; ++t) {
      const LayerPlan& p = layers[t];
      LayerBufs& lb = b.lay[t];
      lb.h_in = prev_h;
      lb.gh_in = prev_gh;
      lb.x = ar.take<T>((size_t)N * p.tp.NX * C);
      lb.gx = p.scalar_src ? nullptr : ar.take<T>((size_t)N * p.tp.NX * C);
      const bool ghosts = (N != NL) && !p.scalar_src;  // exchanged copies of x and of its gradient
      lb.xx = ghosts ? ar.take<T>((size_t)N * p.tp.NX * C) : nullptr;
      lb.gxx = ghosts ? ar.take<T>((size_t)N * p.tp.NX * C) : nullptr;
      if (rt_K) {  // tabulated radial weights: no per-edge activation or weight exists
        lb.H3 = lb.Z1 = lb.Z2 = lb.Z3 = lb.Hact = lb.W = nullptr;
      } else {
        lb.H3 = chunked ? shared_edge[0] : ar.take<T>((size_t)E * kHidden);
        lb.Z1 = chunked ? shared_edge[1] : ar.take<T>((size_t)E * kHidden);
        lb.Z2 = chunked ? shared_edge[2] : ar.take<T>((size_t)E * kHidden);
        lb.Z3 = chunked ? shared_edge[3] : ar.take<T>((size_t)E * kHidden);
        lb.Hact = chunked ? shared_edge[4] : ar.take<T>((size_t)E * kHidden);
        lb.W = chunked ? shared_W : ar.take<T>((size_t)E * p.tp.NP * C);
      }
      lb.M = ar.take<T>((size_t)NL * p.tp.NM * C);
      lb.Gt = ar.take<T>((size_t)NL * (L + 1 + D) * C);
      lb.gGt = ar.take<T>((size_t)NL * (L + 1 + D) * C);
      lb.inv_density = density ? ar.take<T>(NL) : nullptr; lb.gdens = density ? ar.take<T>(NL) : nullptr;
      lb.XY = lb.gXY = lb.Zg = lb.gZg = nullptr;
      if (p.tece) {
        const size_t Es = (size_t)E;
        lb.tKs = ar.take<T>(Es * t_NR * C); lb.tQt = ar.take<T>(Es * t_NR * C); lb.tMw = ar.take<T>(Es * t_NR * 2 * C);
        lb.tKp = ar.take<T>(Es * t_NR * C); lb.tQp = ar.take<T>(Es * t_NR * C);
        lb.tlogit = ar.take<T>(Es * heads); lb.talpha = ar.take<T>(Es * heads);
        lb.tup = ar.take<T>(Es * (t_G + t_NF) * Ca); lb.tglu = ar.take<T>(Es * t_NF * Ca); lb.tcoef = ar.take<T>(Es * t_WN);
        lb.tU = ar.take<T>(Es * t_NF * Ca); lb.tdown = ar.take<T>(Es * t_NR * C);
        lb.tgdown = ar.take<T>(Es * t_NR * C); lb.tgalpha = ar.take<T>(Es * heads); lb.tglogit = ar.take<T>(Es * heads);
        lb.tgcut = ar.take<T>(Es * heads); lb.tgproj = ar.take<T>(Es * 2 * heads); lb.tproj = ar.take<T>(Es * 2 * heads);
        lb.tgQp = ar.take<T>(Es * t_NR * C); lb.tgKp = ar.take<T>(Es * t_NR * C);
        lb.tgKs = ar.take<T>(Es * t_NR * C); lb.tgQt = ar.take<T>(Es * t_NR * C);
        lb.tdxt = ar.take<T>(Es * D * C); lb.tddlen = ar.take<T>(Es);
      }
      if (bilinear) {
        lb.XY = ar.take<T>((size_t)NL * D * 2 * C); lb.gXY = ar.take<T>((size_t)NL * D * 2 * C);
        lb.Zg = ar.take<T>((size_t)NL * p.pb.NP * C); lb.gZg = ar.take<T>((size_t)NL * p.pb.NP * C);
      }
      lb.a = ar.take<T>((size_t)NL * D * C);
      lb.ga = ar.take<T>((size_t)NL * D * C);
      lb.A = ar.take<T>((size_t)NL * D * C);
      lb.gA = ar.take<T>((size_t)NL * D * C);
      lb.B2 = ar.take<T>((size_t)NL * p.pb.NB * C);
      lb.B3 = cfg.correlation >= 3 ? ar.take<T>((size_t)NL * p.pb3.NB * C) : nullptr;
      lb.gB2 = cfg.correlation >= 3 ? ar.take<T>((size_t)NL * p.pb.NB * C) : nullptr;
      lb.As = ar.take<T>((size_t)NL * D * C);
      lb.gAs = ar.take<T>((size_t)NL * D * C);
      lb.gout_s = ar.take<T>((size_t)NL * p.Dout * C);
      lb.hs = p.has_res ? ar.take<T>((size_t)NL * p.Din * C) : nullptr;
      lb.out = ar.take<T>((size_t)NL * p.Dout * C);
      lb.gout = ar.take<T>((size_t)NL * p.Dout * C);
      lb.h_out = ar.take<T>((size_t)N * p.Dout * C);
      lb.gh_out = ar.take<T>((size_t)N * p.Dout * C);
      prev_h = lb.h_out;
      prev_gh = lb.gh_out;
    }
    return ar.used;
  }

  int workspace_bytes(int64_t n_atoms, int64_t n_local, int64_t n_edges, int32_t n_graphs, size_t* bytes) override {
    if (!bytes || n_atoms < 0 || n_local < 0 || n_local > n_atoms || n_edges < 0 || n_graphs < 0) return TACE_ERR_INVALID_ARGUMENT;
    if (n_edges >= (1LL << 31) - 64 || n_atoms >= (1LL << 31) - 64) return TACE_ERR_CAPACITY;
    Arena ar; Bufs b;
    *bytes = layout(ar, b, n_atoms, n_local, n_edges, n_graphs) + 512 + this->stage_layout(n_atoms, n_local, n_edges, n_graphs).total;
    return TACE_OK;
  }

  // ---- GEMM helpers ----------------------------------------------------------------------------
  static void add_problem(GemmBatch<T>& gb, const T* A, long long a_s1, long long a_s2, int q, int K, const T* Bm, int N,
                          T* Cm, long long c_s1, long long c_s2, const T* bias, int accumulate, long long b_gs = 0,
                          long long bias_gs = 0, const int* tile_ptr = nullptr) {
    GemmProblem<T>& p = gb.p[gb.n_problems++];
    p.A = A; p.B = Bm; p.C = Cm; p.bias = bias; p.q = q; p.N = N; p.K = K;
    p.a_s1 = a_s1; p.a_s2 = a_s2; p.c_s1 = c_s1; p.c_s2 = c_s2;
    p.b_group_stride = b_gs; p.bias_group_stride = bias_gs; p.accumulate = accumulate; p.tile_ptr = tile_ptr;
  }
  static GemmBatch<T> plain_batch(long long n_atoms) {
    GemmBatch<T> gb;
    memset(&gb, 0, sizeof(gb));
    gb.n_groups = 1; gb.n_atoms = (int)n_atoms;
    return gb;
  }
  const int* tiles(const Bufs& b, int l) const { return b.tile_ptr + l * (n_el + 1); }

  // One per-rank linear of a launch: rows (atom, m) of A times the [K][N] matrix `wname`;
  // `wname_t` names the same matrix transposed ([N][K]), which is what the tensor-core path reads.
  struct LinSpec {
    const T* A; long long a_s1, a_s2; int q, K;
    std::string wname, wname_t; int N;
    T* Cm; long long c_s1, c_s2; const T* bias;
    int accumulate;  // Cm += instead of Cm =
  };
  // Plain (not per-species) linears: tcgen05 for fp32 models when every shape fits, CUDA cores otherwise.
  cudaError_t run_linear(const std::vector<LinSpec>& specs, long long n_atoms, cudaStream_t s) {
    bool tc = kTensorCore && !specs.empty() && specs.size() <= 4;
    for (const auto& sp : specs) tc = tc && tc_linear_supported(sp.N, sp.K);
    if (tc) {
      TcLinearProblem probs[4];
      for (size_t i = 0; i < specs.size(); ++i) {
        const LinSpec& sp = specs[i];
        probs[i] = {reinterpret_cast<const float*>(sp.A), sp.a_s1, sp.a_s2, sp.q, n_atoms, sp.K, sp.N,
                    reinterpret_cast<const float*>(w(sp.wname_t + "_hi")), reinterpret_cast<const float*>(w(sp.wname_t + "_lo")),
                    reinterpret_cast<float*>(sp.Cm), sp.c_s1, sp.c_s2, reinterpret_cast<const float*>(sp.bias)};
        probs[i].accumulate = sp.accumulate;
      }
      return launch_tc_linear(probs, (int)specs.size(), dev_error, s);
    }
    GemmBatch<T> gb = plain_batch(n_atoms);
    for (const auto& sp : specs)
      add_problem(gb, sp.A, sp.a_s1, sp.a_s2, sp.q, sp.K, w(sp.wname), sp.N, sp.Cm, sp.c_s1, sp.c_s2, sp.bias, sp.accumulate);
    return launch_gemm(gb, n_atoms, s);
  }

  // Per-species linears (the reference's e3nnElementLinear, tace/models/linear.py:377-481).  A holds rows of the
  // species-sorted atoms, so species g owns the contiguous rows [species_ptr[g], species_ptr[g+1]) and uses the g-th
  // matrix of `wname` ([n_el][K][N]); `mapped` sends row a of the result to atom species_perm[a].
  struct SpeciesSpec {
    const T* A; long long a_s1, a_s2; int q, K;
    std::string wname, wname_t; int N;
    T* Cm; long long c_s1, c_s2; const T* bias; bool mapped; int accumulate;
  };
  cudaError_t run_species_linear(const std::vector<SpeciesSpec>& specs, const Bufs& b, long long n_atoms, cudaStream_t s) {
    if (specs.empty()) return cudaSuccess;
    bool tc = kTensorCore && specs.size() <= 4;
    for (const auto& sp : specs) tc = tc && tc_linear_supported(sp.N, sp.K) && sp.mapped == specs[0].mapped;
    if (tc) {
      TcLinearProblem probs[4];
      for (size_t i = 0; i < specs.size(); ++i) {
        const SpeciesSpec& sp = specs[i];
        TcLinearProblem& h = probs[i];
        memset(&h, 0, sizeof(h));
        h.A = reinterpret_cast<const float*>(sp.A); h.a_atom_stride = sp.a_s1; h.a_comp_stride = sp.a_s2; h.q = sp.q;
        h.n_atoms = n_atoms; h.K = sp.K; h.N = sp.N;
        h.Bhi = reinterpret_cast<const float*>(w(sp.wname_t + "_hi")); h.Blo = reinterpret_cast<const float*>(w(sp.wname_t + "_lo"));
        h.C = reinterpret_cast<float*>(sp.Cm); h.c_s1 = sp.c_s1; h.c_s2 = sp.c_s2; h.bias = reinterpret_cast<const float*>(sp.bias);
        h.n_groups = n_el; h.group_ptr = b.species_ptr; h.tile_ptr = b.tc_tile_ptr + (sp.q / 2) * (n_el + 1);
        h.atom_map = sp.mapped ? b.species_perm : nullptr;
        h.b_group_stride = (long long)sp.K * sp.N; h.bias_group_stride = sp.N; h.accumulate = sp.accumulate;
        h.b_tiled = 1;  // the packed per-species hi / lo parts are K-tile-major (read once per pass, straight from DRAM)
      }
      return launch_tc_linear(probs, (int)specs.size(), dev_error, s);
    }
    GemmBatch<T> gb;
    memset(&gb, 0, sizeof(gb));
    gb.n_groups = n_el; gb.group_ptr = b.species_ptr; gb.atom_map = nullptr;
    gb.c_atom_map = specs[0].mapped ? b.species_perm : nullptr;
    for (const auto& sp : specs) {
      if (sp.mapped != specs[0].mapped) return cudaErrorInvalidValue;
      add_problem(gb, sp.A, sp.a_s1, sp.a_s2, sp.q, sp.K, w(sp.wname), sp.N, sp.Cm, sp.c_s1, sp.c_s2, sp.bias, sp.accumulate,
                  (long long)sp.K * sp.N, sp.N, tiles(b, sp.q / 2));
    }
    return launch_gemm(gb, n_atoms, s);
  }

#define CK(expr)                                                                                 \
  do {                                                                                           \
    cudaError_t err__ = (expr);                                                                  \
    if (err__ != cudaSuccess) {                                                                  \
      fprintf(stderr, "tace_b200: CUDA error %s at %s:%d\n", cudaGetErrorString(err__), __FILE__, __LINE__); \
      return TACE_ERR_CUDA;                                                                      \
    }                                                                                            \
  } while (0)

#define CKL(expr) do { CK(expr); ++launches; } while (0)
#define PH(name) phase(name, s)

  // Arguments of the per-edge MLP kernels for layers `ts` over edges [e0, e0 + Ec); row r of every [.][64] buffer is edge e0 + r.
  EdgeArgs<T> edge_range(const EdgeArgs<T>& ea, const Bufs& b, const std::vector<int>& ts, long long e0, long long Ec) const {
    EdgeArgs<T> r = ea;
    r.E = Ec; r.n_layers = (int)ts.size(); r.dlen = ea.dlen + e0; r.ddlen = ea.ddlen + e0;
    r.e_src = ea.e_src + e0; r.e_dst = ea.e_dst + e0;
    if (ea.env) r.env = ea.env + e0;
    if (ea.denv) r.denv = ea.denv + e0;
    for (size_t i = 0; i < ts.size(); ++i) {
      r.mlp[i] = ea.mlp[ts[i]];
      r.Z1[i] = b.lay[ts[i]].Z1;
      r.H1[i] = nh == 1 ? b.lay[ts[i]].H3 : b.lay[ts[i]].Hact;  // activation of the first hidden layer
      r.dH1[i] = dh1_buffer(b.lay[ts[i]]);
    }
    return r;
  }
  // ---- TECE edge block --------------------------------------------------------------------------------------
  // the six SO(2) linears of the block (oam_2026_07_05.py:612-676): channel counts and rows per order on both sides
  struct So2Shape { const char* name; int mm, c_in, c_out, n_in[3], n_out[3]; };
  So2Shape so2_shape(int i) const {
    const int n = L + 1;
    So2Shape s{};
    const int red[3] = {n, n - 1, n - 2}, full[3] = {n, n, n};
    auto set = [&](const char* nm, int mm, int ci, int co, const int* in, const int* out) {
      s.name = nm; s.mm = mm; s.c_in = ci; s.c_out = co;
      for (int m = 0; m < 3; ++m) { s.n_in[m] = in[m]; s.n_out[m] = out[m]; }
    };
    const int up_out[3] = {t_G + n, n, n}, coef_out[3] = {t_np * n * Ca, 0, 0};
    switch (i) {
      case 0: set("key", mmax, C, C, red, red); break;
      case 1: set("query", mmax, C, C, red, red); break;
      case 2: set("up", mmax, 2 * C, Ca, red, up_out); break;
      case 3: set("glu", mmax, 2 * C, Ca, red, full); break;
      case 4: set("coefs", 0, 2 * C, 1, red, coef_out); break;
      default: set("down", mmax, Ca, C, full, red); break;
    }
    return s;
  }
  // GEMM problems of one SO(2) linear over the E edges: `in` [E][in_rows][c_in] -> `out` [E][out_rows][c_out] (forward), or the
  // gradient of the output back to the gradient of the input (backward; `out` is then the input gradient)
  void so2_specs(std::vector<LinSpec>& sp, const std::string& pre, int which, const T* in, int in_rows, T* out, int out_rows, bool backward,
                 int accumulate) const {
    const So2Shape sh = so2_shape(which);
    int off_in = 0, off_out = 0;
    for (int m = 0; m <= sh.mm; ++m) {
      const int K = sh.n_in[m] * sh.c_in, Nn = sh.n_out[m] * sh.c_out;
      const std::string nm = pre + "so2." + sh.name + ".m" + std::to_string(m), nmT = pre + "so2." + sh.name + "T.m" + std::to_string(m);
      if (!backward)
        sp.push_back({in + (long long)off_in * sh.c_in, (long long)in_rows * sh.c_in, K, m ? 2 : 1, K, nm, nmT, Nn,
                      out + (long long)off_out * sh.c_out, (long long)out_rows * sh.c_out, Nn, m == 0 ? w(pre + "so2." + sh.name + ".b") : nullptr, 0});
      else  // `in` holds the gradient of the forward output, `out` receives the gradient of the forward input
        sp.push_back({in + (long long)off_out * sh.c_out, (long long)out_rows * sh.c_out, Nn, m ? 2 : 1, Nn, nmT, nm, K,
                      out + (long long)off_in * sh.c_in, (long long)in_rows * sh.c_in, K, nullptr, accumulate});
      // the order-0 block of the input always spans L + 1 rows (oam_2026_07_05.py:211)
      off_in += (m == 0) ? (L + 1) : 2 * sh.n_in[m];
      off_out += (m == 0) ? sh.n_out[0] : 2 * sh.n_out[m];
    }
  }
  TeceArgs<T> tece_args(const EdgeArgs<T>& ea, const Bufs& b, const LayerBufs& lb, const std::string& pre, const T* x_src, long long NL,
                        long long E) const {
    TeceArgs<T> a;
    memset(&a, 0, sizeof(a));
    a.E = E; a.n_local = (int)NL; a.C = C; a.Ca = Ca; a.L = L; a.mmax = mmax; a.H = heads; a.NR = t_NR; a.NC = t_NC; a.G = t_G;
    a.n_paths = t_np; a.gate_m0 = m0; a.act = edge_act;
    for (int r = 0; r < t_NR; ++r) { a.row_l[r] = t_row_l[r]; a.row_m[r] = t_row_m[r]; a.row_comp[r] = t_row_comp[r]; a.row_scale[r] = T(t_row_scale[r]); }
    for (int q = 0; q < t_np; ++q) { a.p_m1[q] = t_p_m1[q]; a.p_m2[q] = t_p_m2[q]; a.p_m3[q] = t_p_m3[q]; a.p_sum[q] = t_p_sum[q]; a.p_scale[q] = T(t_p_scale[q]); }
    a.rp = ea.rp; a.vec = b.vec; a.dlen = b.dlen; a.env = env_after ? b.env : nullptr;
    a.e_src = b.e_src; a.e_dst = b.e_dst; a.rowptr = b.rowptr_dst;
    a.x = x_src; a.W = lb.W; a.Wg = b.tWg; a.Ks = lb.tKs; a.Qt = lb.tQt; a.Mw = lb.tMw; a.Kp = lb.tKp; a.Qp = lb.tQp;
    a.logit = lb.tlogit; a.alpha = lb.talpha; a.temp = w(pre + "att.temp"); a.rproj_w = w(pre + "att.rw"); a.rproj_b = w(pre + "att.rb");
    a.up = lb.tup; a.glu = lb.tglu; a.coefZ = lb.tcoef; a.U = lb.tU; a.down = lb.tdown; a.M = lb.M;
    a.gM = lb.M; a.gdown = lb.tgdown; a.galpha = lb.tgalpha; a.glogit = lb.tglogit; a.gcut = lb.tgcut; a.gproj = lb.tgproj; a.proj = lb.tproj;
    a.gQp = lb.tgQp; a.gKp = lb.tgKp; a.gKs = lb.tgKs; a.gQt = lb.tgQt; a.gMw = lb.tMw;
    a.gU = lb.tU; a.gup = lb.tup; a.gglu = lb.tglu; a.gcoefZ = lb.tcoef; a.gWg = b.tgWg; a.gvec = b.tgvec;
    a.dxe = b.dxe; a.dxt = lb.tdxt; a.gx = lb.gx; a.ddlen_extra = lb.tddlen;
    return a;
  }
  // forward of the block for one layer: lb.W holds the radial weights, the result lands in lb.M
  int tece_forward(const TeceArgs<T>& ta, const LayerBufs& lb, const std::string& pre, long long E, cudaStream_t s) {
    std::vector<LinSpec> sp;
    CKL(launch_tece(ta, TECE_ROTATE_IN, s));
    so2_specs(sp, pre, 0, lb.tKs, t_NR, lb.tKp, t_NR, false, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    so2_specs(sp, pre, 1, lb.tQt, t_NR, lb.tQp, t_NR, false, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    CKL(launch_tece(ta, TECE_LOGIT, s));
    CKL(launch_tece(ta, TECE_SOFTMAX, s));
    so2_specs(sp, pre, 2, lb.tMw, t_NR, lb.tup, t_G + t_NF, false, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    so2_specs(sp, pre, 3, lb.tMw, t_NR, lb.tglu, t_NF, false, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    so2_specs(sp, pre, 4, lb.tMw, t_NR, lb.tcoef, t_WN, false, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    CKL(launch_tece(ta, TECE_MIX, s));
    so2_specs(sp, pre, 5, lb.tU, t_NF, lb.tdown, t_NR, false, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    CKL(launch_tece(ta, TECE_ROTATE_OUT, s));
    return TACE_OK;
  }
  // backward: lb.M holds dE/d(messages); leaves dE/d(radial weights) in lb.W, the per-edge source rows in dxe, the target part
  // added to lb.gx by the caller's order (source sum first), and this layer's share of dE/d(edge vector) in tgvec / tddlen
  int tece_backward(TeceArgs<T> ta, const Bufs& b, const LayerBufs& lb, const std::string& pre, long long N, long long E, bool first_tece,
                    cudaStream_t s) {
    std::vector<LinSpec> sp;
    CKL(launch_tece(ta, TECE_ROTATE_OUT_BWD, s));
    CKL(launch_tece(ta, TECE_ALPHA_BWD, s));
    CKL(launch_tece(ta, TECE_SOFTMAX_BWD, s));
    CKL(launch_tece(ta, TECE_LOGIT_BWD, s));
    CKL(launch_tece(ta, TECE_EDGE_SCALAR_BWD, s));
    so2_specs(sp, pre, 5, lb.tgdown, t_NF, lb.tU, t_NR, true, 0);   // gU over U
    CKL(run_linear(sp, E, s)); sp.clear();
    CKL(launch_tece(ta, TECE_MIX_BWD, s));                           // gup / gglu / gcoef over their forward buffers
    so2_specs(sp, pre, 2, lb.tup, t_NR, lb.tMw, t_G + t_NF, true, 0);  // gMw over Mw
    CKL(run_linear(sp, E, s)); sp.clear();
    so2_specs(sp, pre, 3, lb.tglu, t_NR, lb.tMw, t_NF, true, 1);
    CKL(run_linear(sp, E, s)); sp.clear();
    so2_specs(sp, pre, 4, lb.tcoef, t_NR, lb.tMw, t_WN, true, 1);
    CKL(run_linear(sp, E, s)); sp.clear();
    so2_specs(sp, pre, 0, lb.tgKp, t_NR, lb.tgKs, t_NR, true, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    so2_specs(sp, pre, 1, lb.tgQp, t_NR, lb.tgQt, t_NR, true, 0);
    CKL(run_linear(sp, E, s)); sp.clear();
    CKL(launch_tece(ta, TECE_ROTATE_IN_BWD, s));
    CKL(launch_segment_sum_rows(b.dxe, b.rowptr_src, b.perm_src, lb.gx, 0, (int)N, D * C, s));
    CKL(launch_tece(ta, TECE_TARGET_SUM, s));
    CKL(launch_tece(ta, TECE_WIGNER_GRAD, s));
    ta.accumulate_gvec = first_tece ? 0 : 1;
    CKL(launch_tece(ta, TECE_WIGNER_BWD, s));
    return TACE_OK;
  }

  DensityArgs<T> density_args(const EdgeArgs<T>& ea, const Bufs& b, const LayerBufs& lb, const std::string& pre, long long NL,
                              long long E) const {
    DensityArgs<T> da;
    memset(&da, 0, sizeof(da));
    da.rowptr_dst = b.rowptr_dst; da.e_dst = b.e_dst; da.dlen = b.dlen; da.rp = ea.rp;
    da.A0 = w(pre + "dA0"); da.w1 = w(pre + "dw1"); da.ab = w(pre + "dab");
    if (mlp_bias) { da.b0 = w(pre + "db0"); da.b1 = w(pre + "db1"); }
    da.use_env = (env_after && density == 1) ? 1 : 0;
    da.n = (int)NL; da.E = E; da.inv_density = lb.inv_density;
    return da;
  }
  // where the backward pass leaves dE/d(first hidden activation): it ping-pongs through the activation buffers
  T* dh1_buffer(const LayerBufs& lb) const { return nh == 3 ? lb.Z3 : nh == 2 ? lb.Hact : lb.H3; }
  // radial MLP hidden layers 8 -> 64 -> 64 -> 64 (tace/models/mlp.py:136-191): the first layer per edge, the
  // two 64 x 64 layers as GEMMs over the edges (all layers of `ts` in one launch), SiLU in between
  int radial_forward(const EdgeArgs<T>& ea, const Bufs& b, const std::vector<int>& ts, long long e0, long long Ec, cudaStream_t s) {
    if (Ec <= 0 || rt_K) return TACE_OK;  // tabulated weights: the radial MLP never runs
    const EdgeArgs<T> er = edge_range(ea, b, ts, e0, Ec);
    CKL(launch_edge_mlp_in(er, s));
    const long long n64 = Ec * kHidden;
    const bool ln = element2;  // LayerNorm before every hidden activation
    for (int j = 0; j < nh; ++j) {  // hidden layer j: activation, then (unless it is the last) the next 64 x 64 layer
      const bool last_hidden = (j == nh - 1);
      for (int t : ts) {
        if (!ln && j == 0) break;  // launch_edge_mlp_in wrote silu(Z1) already
        const LayerBufs& lb = b.lay[t];
        const T* z = j == 0 ? lb.Z1 : j == 1 ? lb.Z2 : lb.Z3;
        T* h = last_hidden ? lb.H3 : lb.Hact;
        if (ln) {
          const std::string pre = "t" + std::to_string(t) + ".ln" + std::to_string(j);
          CKL(launch_ln_silu_fwd(z, w(pre + "g"), w(pre + "b"), h, Ec, s));
        } else {
          CKL(launch_silu(z, h, n64, s));
        }
      }
      if (last_hidden) break;
      std::vector<LinSpec> sp;
      for (int t : ts) {
        const std::string pre = "t" + std::to_string(t) + ".";
        const std::string an = j == 0 ? "A1" : "A2";
        const LayerBufs& lb = b.lay[t];
        sp.push_back({lb.Hact, kHidden, 0, 1, kHidden, pre + an, pre + an + "t", kHidden, j == 0 ? lb.Z2 : lb.Z3, kHidden,
                      0, mlp_bias ? w(pre + (j == 0 ? "b1" : "b2")) : nullptr});
      }
      CKL(run_linear(sp, Ec, s));
    }
    return TACE_OK;
  }
  // back through the hidden layers: lay[t].H3 holds dE/dh3 on entry; ddlen receives dE/d(edge length)
  int radial_backward(const EdgeArgs<T>& ea, const Bufs& b, const std::vector<int>& ts, long long e0, long long Ec, int accumulate,
                      cudaStream_t s) {
    if (Ec <= 0) return TACE_OK;
    if (rt_K) {
      // Tabulated weights: the tensor-product backward passes added their dE/d(edge length) to ddlen already; what is
      // left of this stage is the envelope's own derivative (apply_cutoff = False), once, with the last layer processed.
      const bool last_call = ts.size() > 1 || NL_ == 1 || ts[0] == 0;
      if (!last_call || !ea.denv) return TACE_OK;
      EdgeArgs<T> er = edge_range(ea, b, std::vector<int>{}, e0, Ec);
      er.accumulate_ddlen = 1; er.add_denv = 1;
      CKL(launch_edge_mlp_out(er, s));
      return TACE_OK;
    }
    const long long n64 = Ec * kHidden;
    // gradient buffer chain: H3 -> Hact -> Z3 (three hidden layers), H3 -> Hact (two), H3 (one); the first layer's
    // activation derivative is applied by launch_edge_mlp_out
    const bool ln = element2;
    for (int j = nh - 1; j >= 1; --j) {
      for (int t : ts) {
        const LayerBufs& lb = b.lay[t];
        T* g = (j == nh - 1) ? lb.H3 : lb.Hact;
        if (ln) {
          const std::string pre = "t" + std::to_string(t) + ".ln" + std::to_string(j);
          CKL(launch_ln_silu_bwd(g, j == 1 ? lb.Z2 : lb.Z3, w(pre + "g"), w(pre + "b"), Ec, s));
        } else {
          CKL(launch_silu_grad_mul(g, j == 1 ? lb.Z2 : lb.Z3, n64, s));
        }
      }
      std::vector<LinSpec> sp;
      for (int t : ts) {
        const std::string pre = "t" + std::to_string(t) + ".";
        const std::string an = j == 1 ? "A1" : "A2";
        const LayerBufs& lb = b.lay[t];
        const T* g = (j == nh - 1) ? lb.H3 : lb.Hact;
        T* dst = (j == nh - 1) ? lb.Hact : lb.Z3;
        sp.push_back({g, kHidden, 0, 1, kHidden, pre + an + "t", pre + an, kHidden, dst, kHidden, 0, nullptr});
      }
      CKL(run_linear(sp, Ec, s));
    }
    EdgeArgs<T> er = edge_range(ea, b, ts, e0, Ec);
    if (ln) {  // through the first hidden layer's LayerNorm and activation; launch_edge_mlp_out then starts from dE/dz1
      for (int t : ts) {
        const std::string pre = "t" + std::to_string(t) + ".ln0";
        CKL(launch_ln_silu_bwd(dh1_buffer(b.lay[t]), b.lay[t].Z1, w(pre + "g"), w(pre + "b"), Ec, s));
      }
      er.dz1_given = 1;
    }
    er.accumulate_ddlen = accumulate;
    // the envelope term enters once: with the whole batch in one call, or with the last layer processed (layer 0)
    er.add_denv = (ts.size() > 1 || NL_ == 1 || ts[0] == 0) ? 1 : 0;
    CKL(launch_edge_mlp_out(er, s));
    return TACE_OK;
  }
  // last radial-MLP layer for edges [e0, e0 + Ec): W[e, :] = H3[e, :] @ W3 (forward) or dH3[e, :] = dW[e, :] @ W3^T
  int radial_last(const LayerPlan& p, const LayerBufs& lb, const std::string& pre, long long Ec, bool backward, cudaStream_t s) {
    if (Ec <= 0 || rt_K) return TACE_OK;  // tabulated weights: the radial MLP never runs
    const int NW = p.tp.NP * C;
    if (kTensorCore && NW % 64 == 0) {
      if (!backward)
        CKL(launch_tc_gemm(reinterpret_cast<const float*>(lb.H3), kHidden, reinterpret_cast<const float*>(w(pre + "W3t_hi")),
                           reinterpret_cast<const float*>(w(pre + "W3t_lo")), reinterpret_cast<float*>(lb.W), (long long)NW, (int)Ec,
                           NW, kHidden, dev_error, s, mlp_bias ? reinterpret_cast<const float*>(w(pre + "b3")) : nullptr));
      else
        CKL(launch_tc_gemm(reinterpret_cast<const float*>(lb.W), (long long)NW, reinterpret_cast<const float*>(w(pre + "W3_hi")),
                           reinterpret_cast<const float*>(w(pre + "W3_lo")), reinterpret_cast<float*>(lb.H3), kHidden, (int)Ec,
                           kHidden, NW, dev_error, s));
    } else {
      GemmBatch<T> gb = plain_batch(Ec);
      if (!backward) add_problem(gb, lb.H3, kHidden, 0, 1, kHidden, w(pre + "W3"), NW, lb.W, (long long)NW, 0,
                                 mlp_bias ? w(pre + "b3") : nullptr, 0);
      else add_problem(gb, lb.W, (long long)NW, 0, 1, NW, w(pre + "W3t"), kHidden, lb.H3, kHidden, 0, nullptr, 0);
      CKL(launch_gemm(gb, Ec, s));
    }
    return TACE_OK;
  }
#define CKS(expr) do { const int st__ = (expr); if (st__ != TACE_OK) return st__; } while (0)

  int forward(const TaceBatch* bt, const TaceOutputs* o, void* ws, size_t ws_bytes, cudaStream_t s) override {
    if (!bt || !o || !ws) return TACE_ERR_INVALID_ARGUMENT;
    for (const auto& e : weights)
      if (!e.set) return TACE_ERR_WEIGHTS_MISSING;
    const long long N = bt->n_atoms, NL = bt->n_local, E = bt->n_edges;
    const int B = bt->n_graphs;
    if (N < 0 || NL < 0 || NL > N || E < 0 || B <= 0 || !bt->species || !bt->graph_ptr || (E > 0 && !bt->edge_index))
      return TACE_ERR_INVALID_ARGUMENT;
    const bool vec_mode = bt->edge_vector != nullptr;
    if (!vec_mode && E > 0 && (!bt->positions || !bt->lattice || !bt->edge_shifts)) return TACE_ERR_INVALID_ARGUMENT;
    // ghost atoms need a feature exchange between layers (tace_set_exchange)
    if (NL != N && NL_ > 1 && (!exchange_fn || !vec_mode)) return TACE_ERR_UNSUPPORTED_CONFIG;
    if ((reinterpret_cast<uintptr_t>(ws) & 255) != 0) return TACE_ERR_INVALID_ARGUMENT;
    Arena ar; ar.base = static_cast<unsigned char*>(ws);
    Bufs b;
    if (layout(ar, b, N, NL, E, B) > ws_bytes) return TACE_ERR_CAPACITY;
    debug.clear();
    const bool need_grad = o->forces || o->virials || o->stress || o->edge_forces;

    phase_used = 0;
    if (NL == 0) {
      // A rank that owns no atom (a block of vacuum in a domain decomposition): nothing to evaluate, results are
      // zero, but the exchange callback still runs once per exchanged layer and direction, with zero rows, so that
      // the point-to-point pattern of the other ranks stays matched.
      if (o->energy) CKL(launch_fill_zero(static_cast<T*>(o->energy), (long long)B, s));
      if (o->forces) CKL(launch_fill_zero(static_cast<T*>(o->forces), 3 * N, s));
      if (o->virials) CKL(launch_fill_zero(static_cast<T*>(o->virials), 9LL * B, s));
      if (o->stress) CKL(launch_fill_zero(static_cast<T*>(o->stress), 9LL * B, s));
      if (o->edge_forces) CKL(launch_fill_zero(static_cast<T*>(o->edge_forces), 3 * E, s));
      for (int pass = 0; pass < (need_grad ? 2 : 1); ++pass)
        for (int k = 0; k < NL_; ++k) {
          const int t = pass == 0 ? k : NL_ - 1 - k;
          LayerBufs& lb = b.lay[t];
          const long long row = (long long)layers[t].tp.NX * C;
          if (pass == 0 && lb.xx) {
            CKL(launch_fill_zero(lb.x, N * row, s));
            CKS(exchange_begin(0, lb.x, lb.xx, N, (int)row, s));
            CKS(exchange_join(s));
          }
          if (pass == 1 && lb.gxx) {
            CKL(launch_fill_zero(lb.gx, N * row, s));
            CKS(exchange_begin(1, lb.gx, lb.gxx, N, (int)row, s));
            CKS(exchange_join(s));
          }
        }
      return TACE_OK;
    }
    PH("graph_prep");
    // ---- graph preparation
    GraphPrepArgs gp;
    gp.E = E; gp.n_atoms = (int)N; gp.n_local = (int)NL; gp.n_graphs = B; gp.n_elements = n_el;
    gp.edge_index = bt->edge_index; gp.species = bt->species; gp.graph_ptr = bt->graph_ptr;
    gp.e_src = b.e_src; gp.e_dst = b.e_dst; gp.e_orig = b.e_orig; gp.rowptr_dst = b.rowptr_dst;
    gp.perm_src = b.perm_src; gp.rowptr_src = b.rowptr_src; gp.atom_graph = b.atom_graph;
    gp.species_perm = b.species_perm; gp.species_ptr = b.species_ptr; gp.tile_ptr = b.tile_ptr; gp.tc_tile_ptr = b.tc_tile_ptr;
    gp.temp = b.prep_temp; gp.temp_bytes = b.prep_temp_bytes;
    // edge chunks: one chunk (all atoms) unless the batch exceeds max_chunk_edges
    const bool chunked = E > max_chunk_edges;
    // With an exchange stream the tensor-product passes of the exchanged layers run in two parts: the target atoms none
    // of whose sources is a ghost while the ghost rows travel, the others afterwards (forward), and the other way round
    // for the gradients.  Every target is still summed in one piece, so the numbers do not depend on the schedule.
    const bool overlap = exchange_on_side() && !chunked && NL != N && NL_ > 1;
    gp.split_rows = overlap ? 1 : 0; gp.row_ids = b.row_ids; gp.row_split = b.row_split;
    CKL(launch_graph_prep(gp, s));
    launches += 8 + (overlap ? 2 : 0);  // launch_graph_prep runs nine kernels of its own (eleven) besides the radix sorts
    std::vector<int> chunk_atom{0, (int)NL}, chunk_edge{0, (int)E};
    if (chunked) {
      const int nc = b.n_chunks;
      CKL(launch_chunk_bounds(b.rowptr_dst, (int)NL, max_chunk_edges, nc, b.chunk_atom_ptr, b.chunk_edge_ptr, s));
      chunk_atom.assign(nc + 1, 0); chunk_edge.assign(nc + 1, 0);
      CK(cudaMemcpyAsync(chunk_atom.data(), b.chunk_atom_ptr, sizeof(int) * (nc + 1), cudaMemcpyDeviceToHost, s));
      CK(cudaMemcpyAsync(chunk_edge.data(), b.chunk_edge_ptr, sizeof(int) * (nc + 1), cudaMemcpyDeviceToHost, s));
      CK(cudaStreamSynchronize(s));
      for (int c = 0; c < nc; ++c)
        if (chunk_edge[c + 1] - chunk_edge[c] > b.chunk_rows) return TACE_ERR_CAPACITY;  // an atom with more than kChunkSlack edges
      if (need_grad && NL_ > 1) {
        CKL(launch_chunk_src_sort(b.e_src, E, (int)N, b.chunk_edge_ptr, nc, b.keys_cs, b.perm_cs, b.prep_temp, b.prep_temp_bytes, s));
        ++launches;
      }
    }
    const int n_chunks = (int)chunk_atom.size() - 1;
    PH("edge_fwd");

    // ---- edge features
    EdgeArgs<T> ea;
    memset(&ea, 0, sizeof(ea));
    ea.L = L; ea.n_layers = NL_; ea.E = E;
    ea.e_src = b.e_src; ea.e_dst = b.e_dst; ea.e_orig = b.e_orig;
    ea.positions = static_cast<const T*>(bt->positions); ea.lattice = static_cast<const T*>(bt->lattice);
    ea.atom_graph = b.atom_graph; ea.shifts = static_cast<const T*>(bt->edge_shifts);
    ea.edge_vector = static_cast<const T*>(bt->edge_vector);
    {
      // the radial parameters travel by value inside the kernel arguments
      for (int k = 0; k < kNumBessel; ++k) ea.rp.w[k] = host_bessel[k];
      ea.rp.pref = host_bessel[kNumBessel];
      ea.rp.rc = T(cfg.cutoff); ea.rp.p = cfg.envelope_p;
    }
    for (int t = 0; t < NL_; ++t) {
      const std::string pre = "t" + std::to_string(t) + ".";
      memset(&ea.mlp[t], 0, sizeof(ea.mlp[t]));
      ea.mlp[t].A0 = w(pre + "A0");
      if (mlp_bias) ea.mlp[t].b0 = w(pre + "b0");
      if (element2) { ea.mlp[t].tbl_dst = w(pre + "tdst"); ea.mlp[t].tbl_src = w(pre + "tsrc"); }
      ea.Z1[t] = b.lay[t].Z1;
      ea.dH1[t] = dh1_buffer(b.lay[t]);
    }
    ea.rp.env_after_mlp = env_after ? 1 : 0;
    ea.species = bt->species;
    ea.env = b.env; ea.denv = b.denv; ea.add_denv = 1;
    ea.dlen = b.dlen; ea.ddlen = b.ddlen;
    ea.vec = b.vec; ea.Y = b.Y; ea.dY = b.dY; ea.g = b.g; ea.edge_forces = static_cast<T*>(o->edge_forces);
    CKL(launch_edge_fwd(ea, s));
    std::vector<int> all_layers;
    for (int t = 0; t < NL_; ++t) all_layers.push_back(t);
    PH("radial_mlp_fwd");
    if (!chunked) CKS(radial_forward(ea, b, all_layers, 0, E, s));  // all layers at once; chunked passes do it per layer and chunk
    debug.push_back({"Y", b.Y, (long long)D * E});
    debug.push_back({"vec", b.vec, 3 * E});

    // ---- layers, forward
    bool wigner_done = false, tece_seen = false;
    PH("embed");
    CKL(launch_species_gather(w("emb"), bt->species, b.lay[0].h_in, (int)N, C, s));
    for (int t = 0; t < NL_; ++t) {
      const LayerPlan& p = layers[t];
      LayerBufs& lb = b.lay[t];
      const std::string pre = "t" + std::to_string(t) + ".";
      const std::string ts = std::to_string(t);
      PH(("t" + ts + ".fwd.linear_up").c_str());
      const long long n_up = p.scalar_src ? N : NL;  // layer 0 embeds every atom; later layers own only local rows
      {  // linear_up
        std::vector<LinSpec> sp;
        for (int l : p.in_ls)
          sp.push_back({lb.h_in + (long long)l * l * C, (long long)p.Din * C, C, 2 * l + 1, C, pre + "up.l" + std::to_string(l),
                        pre + "upT.l" + std::to_string(l), C, lb.x + (long long)l * l * C, (long long)p.tp.NX * C, C,
                        l == 0 ? w(pre + "up.b") : nullptr});
        CKL(run_linear(sp, n_up, s));
      }
      const T* x_src = lb.x;
      const bool split = overlap && lb.xx && !p.tece;
      if (lb.xx) {
        // Ghost rows of x are copies of rows owned elsewhere: zero them, let the caller's exchange fill
        // them (lmp_data.forward_exchange in the reference, tace/models/lammps.py:82-129).
        CKL(launch_fill_zero(lb.x + NL * p.tp.NX * C, (N - NL) * p.tp.NX * C, s));
        CKS(exchange_begin(0, lb.x, lb.xx, N, p.tp.NX * C, s));
        if (!split) CKS(exchange_join(s));
        x_src = lb.xx;
      }
      for (int c = 0; c < n_chunks; ++c) {
        const long long e0 = chunk_edge[c], Ec = chunk_edge[c + 1] - e0;
        const int a0 = chunk_atom[c], na = chunk_atom[c + 1] - a0;
        if (chunked) {
          PH("radial_mlp_fwd");
          CKS(radial_forward(ea, b, std::vector<int>{t}, e0, Ec, s));
        }
        PH(("t" + ts + ".fwd.radial_gemm").c_str());
        CKS(radial_last(p, lb, pre, Ec, false, s));
        PH(("t" + ts + ".fwd.tp").c_str());
        if (p.tece) {  // the edge block instead of the tensor product (whole batch only)
          if (chunked) return TACE_ERR_CAPACITY;
          const TeceArgs<T> tc = tece_args(ea, b, lb, pre, x_src, NL, E);
          if (!wigner_done) { CKL(launch_tece(tc, TECE_WIGNER, s)); wigner_done = true; }
          CKS(tece_forward(tc, lb, pre, E, s));
          continue;
        }
        TPArgs<T> ta;
        memset(&ta, 0, sizeof(ta));
        ta.L = L; ta.scalar_src = p.scalar_src; ta.Lin = Ln; ta.C = C; ta.n_seg = na; ta.rowptr = b.rowptr_dst + a0;
        ta.e_src = b.e_src; ta.Y = b.Y; ta.W = lb.W; ta.x = x_src; ta.M = lb.M + (long long)a0 * p.tp.NM * C; ta.e_base = e0;
        ta.env = b.env;
        if (rt_K) { ta.rtab = w(pre + "rtab"); ta.rt_K = rt_K; ta.rt_inv_h = T(rt_K) / T(cfg.cutoff); ta.dlen = b.dlen; }
        if (split) {  // targets that read owned rows only (final in x itself); the others once the ghost rows have arrived
          ta.x = lb.x; ta.row_ids = b.row_ids; ta.row_split = b.row_split + 1; ta.row_part = 0;
          CKL(launch_tp_fwd(ta, s));
          CKS(exchange_join(s));
          ta.x = lb.xx; ta.row_part = 1;
        }
        CKL(launch_tp_fwd(ta, s));
      }
      debug.push_back({"x" + ts, lb.x, N * p.tp.NX * C});
      debug.push_back({"M" + ts, lb.M, NL * p.tp.NM * C});
      PH(("t" + ts + ".fwd.node").c_str());
      {  // linear_down (1/avg_num_neighbors folded into the weights)
        std::vector<LinSpec> sp;
        for (int l = 0; l <= L; ++l) {
          const int K = p.tp.k[l] * C;
          const int Nout = (l == 0) ? (L + 1 + m0) * C : C;
          T* dst = (l == 0) ? lb.Gt : lb.Gt + (long long)(L + m0 + l * l) * C;
          sp.push_back({lb.M + (long long)p.tp.base[l] * C, (long long)p.tp.NM * C, K, 2 * l + 1, K, pre + "down.l" + std::to_string(l),
                        pre + "downT.l" + std::to_string(l), Nout, dst, (long long)(L + 1 + D) * C, C,
                        l == 0 ? w(pre + "down.b") : nullptr});
        }
        CKL(run_linear(sp, NL, s));
      }
      if (density) {  // learned normalisation instead of the constant folded into the weights
        const DensityArgs<T> da = density_args(ea, b, lb, pre, NL, E);
        CKL(launch_density_fwd(da, s));
        CKL(launch_scale_rows(lb.Gt, lb.inv_density, NL, (L + m0 + D) * C, (long long)(L + 1 + D) * C, s));
      }
      CKL(launch_gate_fwd(lb.Gt, lb.a, (int)NL, L, C, m0, s));
      {
        std::vector<LinSpec> sp;
        for (int l = 0; l <= L; ++l)
          sp.push_back({lb.a + (long long)l * l * C, (long long)D * C, C, 2 * l + 1, C, pre + "nl.l" + std::to_string(l),
                        pre + "nlT.l" + std::to_string(l), C, lb.A + (long long)l * l * C, (long long)D * C, C,
                        l == 0 ? w(pre + "nl.b") : nullptr});
        CKL(run_linear(sp, NL, s));
      }
      debug.push_back({"A" + ts, lb.A, NL * D * C});
      // per-species part in species-sorted space: gather A, product basis, coefficient linears scatter into `out`
      CKL(launch_gather_rows(lb.A, b.species_perm, lb.As, NL, D * C, s));
      if (bilinear) {
        std::vector<LinSpec> sp;
        for (int l = 0; l <= L; ++l)
          sp.push_back({lb.As + (long long)l * l * C, (long long)D * C, C, 2 * l + 1, C, pre + "pu.l" + std::to_string(l),
                        pre + "puT.l" + std::to_string(l), 2 * C, lb.XY + (long long)l * l * 2 * C, (long long)D * 2 * C, 2 * C,
                        l == 0 ? w(pre + "pu.b") : nullptr});
        CKL(run_linear(sp, NL, s));
        sp.clear();
        sp.push_back({lb.As, (long long)D * C, C, 1, C, pre + "pg", pre + "pgT", p.pb.NP * C, lb.Zg, (long long)p.pb.NP * C, 0,
                      w(pre + "pg.b")});
        CKL(run_linear(sp, NL, s));
        CKL(launch_pbl_fwd(lb.XY, lb.Zg, lb.B2, (int)NL, L, p.pb_lout, C, s));
      } else if (cfg.correlation >= 2) {
        CKL(launch_pb_fwd(lb.As, lb.B2, (int)NL, L, p.pb_lout, C, s));
      }
      if (cfg.correlation >= 3) CKL(launch_pb3_fwd(lb.As, lb.B2, lb.B3, (int)NL, L, p.last ? -1 : Ln, C, s));
      {
        std::vector<SpeciesSpec> sp;
        for (int l : p.out_ls)
          sp.push_back({bilinear ? lb.XY + (long long)l * l * 2 * C : lb.As + (long long)l * l * C, (long long)D * C * (bilinear ? 2 : 1),
                        (long long)C * (bilinear ? 2 : 1), 2 * l + 1, C, pre + "c0.l" + std::to_string(l),
                        pre + "c0T.l" + std::to_string(l), C, lb.out + (long long)l * l * C, (long long)p.Dout * C, C,
                        l == 0 ? w(pre + "c.b") : nullptr, true, 0});
        CKL(run_species_linear(sp, b, NL, s));
        if (cfg.correlation >= 2) {
          sp.clear();
          for (size_t i = 0; i < p.out_ls.size(); ++i) {
            const int l = p.out_ls[i];
            const int K = p.pb.k[i] * C;
            sp.push_back({lb.B2 + (long long)p.pb.base[i] * C, (long long)p.pb.NB * C, K, 2 * l + 1, K, pre + "c1.l" + std::to_string(l),
                          pre + "c1T.l" + std::to_string(l), C, lb.out + (long long)l * l * C, (long long)p.Dout * C, C, nullptr, true, 1});
          }
          CKL(run_species_linear(sp, b, NL, s));
        }
        if (cfg.correlation >= 3) {
          sp.clear();
          for (size_t i = 0; i < p.out_ls.size(); ++i) {
            const int l = p.out_ls[i];
            const int K = p.pb3.k[i] * C;
            sp.push_back({lb.B3 + (long long)p.pb3.base[i] * C, (long long)p.pb3.NB * C, K, 2 * l + 1, K, pre + "c2.l" + std::to_string(l),
                          pre + "c2T.l" + std::to_string(l), C, lb.out + (long long)l * l * C, (long long)p.Dout * C, C, nullptr, true, 1});
          }
          CKL(run_species_linear(sp, b, NL, s));
        }
      }
      {
        std::vector<LinSpec> sp;
        for (int l : p.out_ls)
          sp.push_back({lb.out + (long long)l * l * C, (long long)p.Dout * C, C, 2 * l + 1, C, pre + "lin.l" + std::to_string(l),
                        pre + "linT.l" + std::to_string(l), C, lb.h_out + (long long)l * l * C, (long long)p.Dout * C, C,
                        l == 0 ? w(pre + "lin.b") : nullptr});
        CKL(run_linear(sp, NL, s));
      }
      if (p.has_res && res_identity) {  // tace/models/_e3nn/residual.py:216-250: the ranks the output keeps, copied over
        CKL(launch_add_rows(lb.h_out, (long long)p.Dout * C, lb.h_in, (long long)p.Din * C, NL, p.Dout * C, s));
      } else if (p.has_res) {  // per-species skip connection from the layer input
        CKL(launch_gather_rows(lb.h_in, b.species_perm, lb.hs, NL, p.Din * C, s));
        std::vector<SpeciesSpec> sp;
        for (int l : p.out_ls)
          sp.push_back({lb.hs + (long long)l * l * C, (long long)p.Din * C, C, 2 * l + 1, C, pre + "res.l" + std::to_string(l),
                        pre + "resT.l" + std::to_string(l), C, lb.h_out + (long long)l * l * C, (long long)p.Dout * C, C,
                        l == 0 ? w(pre + "res.b") : nullptr, true, 1});
        CKL(run_species_linear(sp, b, NL, s));
      }
      debug.push_back({"h" + std::to_string(t + 1), lb.h_out, NL * p.Dout * C});
    }

    // ---- read-out
    PH("readout");
    LayerBufs& top = b.lay[NL_ - 1];
    ReadoutArgs<T> ra;
    memset(&ra, 0, sizeof(ra));
    ra.h = top.h_out; ra.hs = (long long)layers[NL_ - 1].Dout * C; ra.W1 = w("ro.W1"); ra.W2 = w("ro.W2");
    ra.scale = w("scale"); ra.e0 = w("e0"); ra.species = bt->species; ra.atom_graph = b.atom_graph;
    ra.graph_ptr = bt->graph_ptr; ra.rowptr_dst = b.rowptr_dst; ra.node_energy = static_cast<T*>(o->node_energy);
    ra.e_scaled = b.e_scaled; ra.gh = need_grad ? top.gh_out : nullptr; ra.n = (int)NL; ra.C = C; ra.H = H;
    ra.fidelity = bt->fidelity; ra.n_el = n_el;
    ZblArgs<T> za;
    memset(&za, 0, sizeof(za));
    if (zbl) {  // pair repulsion per atom, summed over the incoming edges
      za.rowptr_dst = b.rowptr_dst; za.e_src = b.e_src; za.e_dst = b.e_dst; za.species = bt->species; za.dlen = b.dlen;
      za.z = w("zbl.z"); za.rcov = w("zbl.rcov"); za.par = w("zbl.par"); za.p = cfg.envelope_p; za.n = (int)NL; za.E = E;
      za.node = b.zbl_node;
      CKL(launch_zbl_fwd(za, s));
      ra.zbl = b.zbl_node; ra.zbl_after = (zbl == 2);
      ra.factor = b.ro_factor;
    }
    if (cfg.use_alllayer) {  // linear read-outs of the layers below the last
      ra.n_extra = NL_ - 1;
      for (int t = 0; t + 1 < NL_; ++t) {
        ra.extra_h[t] = b.lay[t].h_out; ra.extra_hs[t] = (long long)layers[t].Dout * C; ra.extra_w[t] = w("ro.lin" + std::to_string(t));
      }
      ra.factor = b.ro_factor;
    }
    CKL(launch_readout(ra, s));
    if (o->energy) {
      CKL(launch_graph_energy(b.e_scaled, w("e0"), bt->species, bt->graph_ptr, bt->fidelity, n_el, static_cast<T*>(o->energy), B, NL,
                              b.energy_partial, s));
      if (graph_energy_slices(NL, B) > 1) ++launches;  // the slice sums are added by a second kernel
    }
    if (!need_grad) { PH("end"); return TACE_OK; }

    // ---- layers, backward
    for (int t = NL_ - 1; t >= 0; --t) {
      const LayerPlan& p = layers[t];
      LayerBufs& lb = b.lay[t];
      const std::string pre = "t" + std::to_string(t) + ".";
      const std::string ts = std::to_string(t);
      PH(("t" + ts + ".bwd.node").c_str());
      if (cfg.use_alllayer && t + 1 < NL_)  // this layer's own linear read-out, on top of what the layer above sent down
        CKL(launch_readout_linear_bwd(lb.gh_out, (long long)p.Dout * C, b.ro_factor, w("ro.lin" + ts), b.atom_graph, bt->fidelity,
                                      (int)NL, C, s));
      {  // through the final linear
        std::vector<LinSpec> sp;
        for (int l : p.out_ls)
          sp.push_back({lb.gh_out + (long long)l * l * C, (long long)p.Dout * C, C, 2 * l + 1, C, pre + "linT.l" + std::to_string(l),
                        pre + "lin.l" + std::to_string(l), C, lb.gout + (long long)l * l * C, (long long)p.Dout * C, C, nullptr});
        CKL(run_linear(sp, NL, s));
      }
      // through the per-species coefficients and the product basis, in species-sorted space
      CKL(launch_gather_rows(lb.gout, b.species_perm, lb.gout_s, NL, p.Dout * C, s));
      if (bilinear) CKL(launch_fill_zero(lb.gXY, NL * D * 2 * C, s));
      else if ((int)p.out_ls.size() != L + 1) CKL(launch_fill_zero(lb.gAs, NL * D * C, s));
      {
        std::vector<SpeciesSpec> sp;
        for (int l : p.out_ls)
          sp.push_back({lb.gout_s + (long long)l * l * C, (long long)p.Dout * C, C, 2 * l + 1, C, pre + "c0T.l" + std::to_string(l),
                        pre + "c0.l" + std::to_string(l), C, bilinear ? lb.gXY + (long long)l * l * 2 * C : lb.gAs + (long long)l * l * C,
                        (long long)D * C * (bilinear ? 2 : 1), (long long)C * (bilinear ? 2 : 1), nullptr, false, 0});
        CKL(run_species_linear(sp, b, NL, s));
        if (cfg.correlation >= 2) {
          // gradient of the second-order basis: written over B2 itself, or into gB2 when the third order still needs B2
          T* g2 = cfg.correlation >= 3 ? lb.gB2 : lb.B2;
          if (cfg.correlation >= 3) {
            CKL(launch_fill_zero(lb.gB2, NL * p.pb.NB * C, s));  // ranks above the output ranks only receive third-order terms
            sp.clear();
            for (size_t i = 0; i < p.out_ls.size(); ++i) {
              const int l = p.out_ls[i];
              const int K = p.pb3.k[i] * C;
              sp.push_back({lb.gout_s + (long long)l * l * C, (long long)p.Dout * C, C, 2 * l + 1, C, pre + "c2T.l" + std::to_string(l),
                            pre + "c2.l" + std::to_string(l), K, lb.B3 + (long long)p.pb3.base[i] * C, (long long)p.pb3.NB * C, K,
                            nullptr, false, 0});
            }
            CKL(run_species_linear(sp, b, NL, s));  // B3 now holds its gradient
          }
          sp.clear();
          for (size_t i = 0; i < p.out_ls.size(); ++i) {
            const int l = p.out_ls[i];
            const int K = p.pb.k[i] * C;
            sp.push_back({lb.gout_s + (long long)l * l * C, (long long)p.Dout * C, C, 2 * l + 1, C, pre + "c1T.l" + std::to_string(l),
                          pre + "c1.l" + std::to_string(l), K, g2 + (long long)p.pb.base[i] * C, (long long)p.pb.NB * C, K, nullptr,
                          false, 0});
          }
          CKL(run_species_linear(sp, b, NL, s));
          if (cfg.correlation >= 3) {
            CKL(launch_pb3_bwd(lb.As, lb.B2, lb.B3, lb.gB2, lb.gAs, (int)NL, L, p.last ? -1 : Ln, C, s));
            ++launches;
          }
          if (bilinear) {  // back through the gated product, then through the product's own linear_up
            CKL(launch_pbl_bwd(lb.XY, lb.Zg, g2, lb.gXY, lb.gZg, (int)NL, L, p.pb_lout, C, s));
            std::vector<LinSpec> lp;
            for (int l = 0; l <= L; ++l)
              lp.push_back({lb.gXY + (long long)l * l * 2 * C, (long long)D * 2 * C, 2 * C, 2 * l + 1, 2 * C, pre + "puT.l" + std::to_string(l),
                            pre + "pu.l" + std::to_string(l), C, lb.gAs + (long long)l * l * C, (long long)D * C, C, nullptr});
            CKL(run_linear(lp, NL, s));
            lp.clear();
            lp.push_back({lb.gZg, (long long)p.pb.NP * C, 0, 1, p.pb.NP * C, pre + "pgT", pre + "pg", C, lb.gAs, (long long)D * C, 0,
                          nullptr, 1});
            CKL(run_linear(lp, NL, s));
          } else {
            CKL(launch_pb_bwd(lb.As, g2, lb.gAs, (int)NL, L, p.pb_lout, C, s));
          }
        }
      }
      CKL(launch_scatter_rows(lb.gAs, b.species_perm, lb.gA, NL, D * C, s));
      {
        std::vector<LinSpec> sp;
        for (int l = 0; l <= L; ++l)
          sp.push_back({lb.gA + (long long)l * l * C, (long long)D * C, C, 2 * l + 1, C, pre + "nlT.l" + std::to_string(l),
                        pre + "nl.l" + std::to_string(l), C, lb.ga + (long long)l * l * C, (long long)D * C, C, nullptr});
        CKL(run_linear(sp, NL, s));
      }
      CKL(launch_gate_bwd(lb.Gt, lb.ga, lb.gGt, (int)NL, L, C, m0, s));
      if (density)  // d / d density_i, and the gradient of the unscaled linear_down output
        CKL(launch_density_node_bwd(lb.gGt, lb.Gt, lb.inv_density, lb.gdens, NL, (L + m0 + D) * C, (long long)(L + 1 + D) * C, s));
      {  // through linear_down; the gradient of the messages overwrites the messages
        std::vector<LinSpec> sp;
        for (int l = 0; l <= L; ++l) {
          const int Nk = p.tp.k[l] * C;
          const int Kin = (l == 0) ? (L + 1 + m0) * C : C;
          const T* src = (l == 0) ? lb.gGt : lb.gGt + (long long)(L + m0 + l * l) * C;
          sp.push_back({src, (long long)(L + 1 + D) * C, C, 2 * l + 1, Kin, pre + "downT.l" + std::to_string(l),
                        pre + "down.l" + std::to_string(l), Nk, lb.M + (long long)p.tp.base[l] * C, (long long)p.tp.NM * C, Nk, nullptr});
        }
        CKL(run_linear(sp, NL, s));
      }
      // edge pass: gradients of the per-edge weights (in place over W), of the angular features and,
      // per edge, of the source features
      if (chunked && !p.scalar_src) CKL(launch_fill_zero(lb.gx, N * p.tp.NX * C, s));  // chunks add their shares
      for (int c = 0; c < n_chunks; ++c) {
        const long long e0 = chunk_edge[c], Ec = chunk_edge[c + 1] - e0;
        const int a0 = chunk_atom[c], na = chunk_atom[c + 1] - a0;
        if (chunked) {  // the per-edge activations and weights of this chunk were not kept: recompute them
          PH("radial_mlp_fwd");
          CKS(radial_forward(ea, b, std::vector<int>{t}, e0, Ec, s));
          PH(("t" + ts + ".fwd.radial_gemm").c_str());
          CKS(radial_last(p, lb, pre, Ec, false, s));
        }
        PH(("t" + ts + ".bwd.tp").c_str());
        if (p.tece) {
          if (t == NL_ - 1) {  // no tensor product above to initialise the accumulators of the layers below
            CKL(launch_fill_zero(b.dY, E * D, s));
            if (b.denv) CKL(launch_fill_zero(b.denv, E, s));
          }
          const TeceArgs<T> tc = tece_args(ea, b, lb, pre, lb.xx ? lb.xx : lb.x, NL, E);
          CKS(tece_backward(tc, b, lb, pre, N, E, !tece_seen, s));
          tece_seen = true;
          PH(("t" + ts + ".bwd.radial_gemm").c_str());
          CKS(radial_last(p, lb, pre, Ec, true, s));
          continue;
        }
        TPArgs<T> ta;
        memset(&ta, 0, sizeof(ta));
        ta.L = L; ta.scalar_src = p.scalar_src; ta.Lin = Ln; ta.C = C; ta.e_src = b.e_src; ta.Y = b.Y;
        ta.W = lb.W; ta.x = lb.xx ? lb.xx : lb.x; ta.gM = lb.M + (long long)a0 * p.tp.NM * C; ta.n_seg = na;
        ta.rowptr = b.rowptr_dst + a0; ta.dW = lb.W; ta.dY = b.dY; ta.e_base = e0;
        ta.accumulate_dY = (t != NL_ - 1); ta.dxe = p.scalar_src ? nullptr : b.dxe;
        ta.env = b.env; ta.denv = b.denv; ta.accumulate_denv = (t != NL_ - 1);
        if (rt_K) {
          ta.rtab = w(pre + "rtab"); ta.rt_K = rt_K; ta.rt_inv_h = T(rt_K) / T(cfg.cutoff); ta.dlen = b.dlen;
          ta.dW = nullptr; ta.ddlen = b.ddlen; ta.accumulate_ddlen = (t != NL_ - 1);
        }
        if (overlap && lb.gxx) {
          // Targets with ghost sources first: the per-source sums of the ghost rows are what the owners of those atoms
          // wait for.  While they travel the other targets follow; the sums over owned sources land in the owned rows of
          // xx (x itself still holds those rows, and nothing reads xx any more), to be added to the arrivals after the join.
          const int row = p.tp.NX * C;
          TPArgs<T> tb = ta;
          tb.row_ids = b.row_ids; tb.row_split = b.row_split + 1; tb.row_part = 1;
          CKL(launch_tp_bwd(tb, s));
          PH(("t" + ts + ".bwd.src_sum").c_str());
          CKL(launch_fill_zero(lb.gx, NL * row, s));
          CKL(launch_segment_sum_rows(b.dxe, b.rowptr_src, b.perm_src, lb.gx, (int)NL, (int)(N - NL), row, s));
          CKS(exchange_begin(1, lb.gx, lb.gxx, N, row, s));
          PH(("t" + ts + ".bwd.tp").c_str());
          ta.x = lb.x; ta.row_ids = b.row_ids; ta.row_split = b.row_split + 1; ta.row_part = 0;
          CKL(launch_tp_bwd(ta, s));
          PH(("t" + ts + ".bwd.src_sum").c_str());
          CKL(launch_segment_sum_rows(b.dxe, b.rowptr_src, b.perm_src, lb.xx, 0, (int)NL, row, s));
        } else {
          CKL(launch_tp_bwd(ta, s));
          if (!p.scalar_src) {  // sum the per-edge rows over the edges leaving each source atom
            PH(("t" + ts + ".bwd.src_sum").c_str());
            if (chunked) CKL(launch_chunk_src_sum(b.dxe, b.keys_cs, b.perm_cs, e0, e0 + Ec, (long long)c * N, lb.gx, p.tp.NX * C, s));
            else CKL(launch_segment_sum_rows(b.dxe, b.rowptr_src, b.perm_src, lb.gx, 0, (int)N, p.tp.NX * C, s));
          }
        }
        PH(("t" + ts + ".bwd.radial_gemm").c_str());
        CKS(radial_last(p, lb, pre, Ec, true, s));  // back through the last radial-MLP layer: H3 <- dE/dh3
        if (chunked) {
          PH("radial_mlp_bwd");
          CKS(radial_backward(ea, b, std::vector<int>{t}, e0, Ec, t != NL_ - 1, s));
        }
      }
      if (lb.gxx) {  // gradients that landed on ghost rows go back to their owners (reverse_exchange)
        if (overlap && !p.tece) {  // already on its way: owned rows of gxx = arrivals + this rank's own sums
          CKS(exchange_join(s));
          CKL(launch_add_inplace(lb.gxx, lb.xx, NL * p.tp.NX * C, s));
        } else {
          CKS(exchange_begin(1, lb.gx, lb.gxx, N, p.tp.NX * C, s));
          CKS(exchange_join(s));
        }
      }
      if (!p.scalar_src) {
        PH(("t" + ts + ".bwd.linear_up").c_str());
        std::vector<LinSpec> sp;
        for (int l : p.in_ls)
          sp.push_back({(lb.gxx ? lb.gxx : lb.gx) + (long long)l * l * C, (long long)p.tp.NX * C, C, 2 * l + 1, C,
                        pre + "upT.l" + std::to_string(l), pre + "up.l" + std::to_string(l), C, lb.gh_in + (long long)l * l * C,
                        (long long)p.Din * C, C, nullptr});
        CKL(run_linear(sp, NL, s));
        if (p.has_res && res_identity) {
          CKL(launch_add_rows(lb.gh_in, (long long)p.Din * C, lb.gh_out, (long long)p.Dout * C, NL, p.Dout * C, s));
        } else if (p.has_res) {
          CKL(launch_gather_rows(lb.gh_out, b.species_perm, lb.gout_s, NL, p.Dout * C, s));
          std::vector<SpeciesSpec> sp2;
          for (int l : p.out_ls)
            sp2.push_back({lb.gout_s + (long long)l * l * C, (long long)p.Dout * C, C, 2 * l + 1, C, pre + "resT.l" + std::to_string(l),
                           pre + "res.l" + std::to_string(l), C, lb.gh_in + (long long)l * l * C, (long long)p.Din * C, C, nullptr, true, 1});
          CKL(run_species_linear(sp2, b, NL, s));
        }
      }
    }

    // ---- back to the edge vectors, then forces and virials
    PH("radial_mlp_bwd");
    if (!chunked) CKS(radial_backward(ea, b, all_layers, 0, E, 0, s));  // lay[t].H3 holds dE/dh3 of each layer's radial MLP
    for (int t = 0; t < NL_; ++t)  // the edge blocks' own dependence on the edge lengths (radial projection, cutoff in the softmax)
      if (layers[t].tece) CKL(launch_add_inplace(b.ddlen, b.lay[t].tddlen, E, s));
    if (tece_mask) ea.gvec_extra = b.tgvec;  // and on the edge vectors through the frames
    if (density) {  // the densities' dependence on the edge lengths
      for (int t = 0; t < NL_; ++t) {
        DensityArgs<T> da = density_args(ea, b, b.lay[t], "t" + std::to_string(t) + ".", NL, E);
        da.gdens = b.lay[t].gdens; da.ddlen = b.ddlen;
        CKL(launch_density_bwd(da, s));
      }
    }
    if (zbl) {  // the repulsion's own dependence on the edge lengths
      za.ddlen = b.ddlen; za.factor = (zbl == 1) ? b.ro_factor : nullptr;
      CKL(launch_zbl_bwd(za, s));
    }
    PH("edge_bwd");
    CKL(launch_edge_bwd(ea, s));
    debug.push_back({"g", b.g, 3 * E});
    PH("forces");
    const bool want_virial = (o->virials || o->stress) && !vec_mode;
    ForceArgs<T> fa;
    memset(&fa, 0, sizeof(fa));
    fa.n_atoms = (int)N; fa.n_local = (int)NL; fa.rowptr_dst = b.rowptr_dst; fa.rowptr_src = b.rowptr_src;
    fa.perm_src = b.perm_src; fa.g = b.g; fa.vec = b.vec; fa.forces = static_cast<T*>(o->forces);
    fa.atom_virial = want_virial ? b.atom_virial : nullptr;
    if (fa.forces || fa.atom_virial) CKL(launch_forces(fa, s));
    if (want_virial)
      CKL(launch_graph_virial(b.atom_virial, bt->graph_ptr, static_cast<const T*>(bt->lattice), static_cast<T*>(o->virials),
                             static_cast<T*>(o->stress), B, s));
    PH("end");
    return TACE_OK;
  }

  int64_t debug_read(const char* name, void* dst, int64_t numel, cudaStream_t s) override {
    for (const auto& d : debug) {
      if (d.name == name) {
        const long long n = d.numel < numel ? d.numel : numel;
        if (cudaMemcpyAsync(dst, d.ptr, sizeof(T) * (size_t)n, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return TACE_ERR_CUDA;
        return n;
      }
    }
    return TACE_ERR_INVALID_ARGUMENT;
  }
};

}  // namespace tace

using tace::ModelBase;

struct TaceModel {
  ModelBase* impl;
};

extern "C" {

const char* tace_status_string(int status) {
  switch (status) {
    case TACE_OK: return "ok";
    case TACE_ERR_INVALID_ARGUMENT: return "invalid argument";
    case TACE_ERR_UNSUPPORTED_CONFIG: return "unsupported model configuration";
    case TACE_ERR_CAPACITY: return "capacity exceeded (workspace too small or index range)";
    case TACE_ERR_CUDA: return "CUDA error";
    case TACE_ERR_NO_DEVICE: return "no sm_100 CUDA device";
    case TACE_ERR_UNKNOWN_WEIGHT: return "unknown weight name";
    case TACE_ERR_WEIGHTS_MISSING: return "weights not fully set";
    default: return "unknown status";
  }
}

int tace_create(const TaceConfig* cfg, TaceModel** out) {
  if (!cfg || !out) return TACE_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  if (cfg->L < 1 || cfg->L > 3 || cfg->num_layers < 1 || cfg->num_layers > tace::kMaxLayers || cfg->num_channel < 32 ||
      cfg->num_channel > 256 || (cfg->num_channel & 31) || cfg->num_elements < 1 || cfg->correlation < 1 ||
      cfg->correlation > 3 || cfg->num_bessel != tace::kNumBessel || cfg->mlp_hidden != tace::kHidden ||
      cfg->readout_hidden < 1 || cfg->readout_hidden > 64 || cfg->envelope_p < 2 || !(cfg->cutoff > 0.0) ||
      !(cfg->avg_num_neighbors > 0.0) || (cfg->dtype != TACE_F32 && cfg->dtype != TACE_F64))
    return TACE_ERR_UNSUPPORTED_CONFIG;
  int dev = 0;
  cudaDeviceProp prop;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return TACE_ERR_NO_DEVICE;
  if (prop.major != 10) return TACE_ERR_NO_DEVICE;
  ModelBase* impl = nullptr;
  int st;
  if (cfg->dtype == TACE_F32) {
    auto* m = new (std::nothrow) tace::Model<float>();
    if (!m) return TACE_ERR_CUDA;
    st = m->init(*cfg); impl = m;
  } else {
    auto* m = new (std::nothrow) tace::Model<double>();
    if (!m) return TACE_ERR_CUDA;
    st = m->init(*cfg); impl = m;
  }
  if (st != TACE_OK) { delete impl; return st; }
  *out = new TaceModel{impl};
  return TACE_OK;
}

void tace_destroy(TaceModel* model) {
  if (!model) return;
  model->impl->release_graphs();
  delete model->impl;
  delete model;
}

int tace_weight_count(const TaceModel* model) { return model ? model->impl->weight_count() : TACE_ERR_INVALID_ARGUMENT; }
int tace_weight_info(const TaceModel* model, int index, const char** name, int64_t* numel) {
  return model ? model->impl->weight_info(index, name, numel) : TACE_ERR_INVALID_ARGUMENT;
}
int tace_set_weight(TaceModel* model, const char* name, const void* host_data, int64_t numel) {
  return model ? model->impl->set_weight(name, host_data, numel) : TACE_ERR_INVALID_ARGUMENT;
}
int tace_workspace_bytes(const TaceModel* model, int64_t n_atoms, int64_t n_local, int64_t n_edges, int32_t n_graphs,
                         size_t* bytes) {
  return model ? const_cast<TaceModel*>(model)->impl->workspace_bytes(n_atoms, n_local, n_edges, n_graphs, bytes)
               : TACE_ERR_INVALID_ARGUMENT;
}
int tace_forward(TaceModel* model, const TaceBatch* batch, const TaceOutputs* out, void* workspace, size_t workspace_bytes,
                 tace_stream_t stream) {
  if (!model) return TACE_ERR_INVALID_ARGUMENT;
  return model->impl->forward_entry(batch, out, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}
int tace_set_graph_mode(TaceModel* model, int enable) {
  if (!model) return TACE_ERR_INVALID_ARGUMENT;
  model->impl->graph_mode = enable != 0;
  if (!enable) model->impl->release_graphs();
  return TACE_OK;
}
int tace_set_chunk_edges(TaceModel* model, int64_t max_edges) {
  if (!model || max_edges < 1024) return TACE_ERR_INVALID_ARGUMENT;
  model->impl->max_chunk_edges = max_edges;
  model->impl->release_graphs();
  return TACE_OK;
}
int64_t tace_graph_replays(const TaceModel* model) { return model ? model->impl->graph_replays : TACE_ERR_INVALID_ARGUMENT; }
int tace_set_exchange_sync(TaceModel* model, int host_sync) {
  if (!model || !model->impl) return TACE_ERR_INVALID_ARGUMENT;
  model->impl->exchange_sync = host_sync != 0;
  return TACE_OK;
}

int tace_set_exchange_stream(TaceModel* model, tace_stream_t stream) {
  if (!model || !model->impl) return TACE_ERR_INVALID_ARGUMENT;
  model->impl->exchange_stream = static_cast<cudaStream_t>(stream);
  return TACE_OK;
}

int tace_set_exchange(TaceModel* model, tace_exchange_fn fn, void* user) {
  if (!model) return TACE_ERR_INVALID_ARGUMENT;
  model->impl->exchange_fn = fn;
  model->impl->exchange_user = user;
  return TACE_OK;
}
int tace_device_error(TaceModel* model, int32_t* code) {
  if (!model || !code) return TACE_ERR_INVALID_ARGUMENT;
  int v = 0;
  if (cudaMemcpy(&v, model->impl->dev_error, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return TACE_ERR_CUDA;
  if (v != 0 && cudaMemset(model->impl->dev_error, 0, sizeof(int)) != cudaSuccess) return TACE_ERR_CUDA;
  *code = v;
  return TACE_OK;
}
int64_t tace_launch_count(const TaceModel* model) { return model ? model->impl->launches : TACE_ERR_INVALID_ARGUMENT; }
int tace_profile_enable(TaceModel* model, int enable) {
  if (!model) return TACE_ERR_INVALID_ARGUMENT;
  model->impl->profile = enable != 0;
  model->impl->phase_used = 0;
  return TACE_OK;
}
int tace_profile_count(const TaceModel* model) { return model ? model->impl->phase_count() : TACE_ERR_INVALID_ARGUMENT; }
int tace_profile_read(TaceModel* model, int index, const char** name, float* ms) {
  if (!model || !name || !ms) return TACE_ERR_INVALID_ARGUMENT;
  return model->impl->phase_read(index, name, ms);
}
int64_t tace_debug_read(TaceModel* model, const char* name, void* dst, int64_t numel, tace_stream_t stream) {
  if (!model || !name || !dst) return TACE_ERR_INVALID_ARGUMENT;
  return model->impl->debug_read(name, dst, numel, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
