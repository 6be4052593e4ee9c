// FP32-accurate dense GEMM on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), used for
// the last layer of the radial MLP and its transpose (the reference's mlpLinear torch.mm,
// tace/models/linear.py:267-276, which produces the per-edge tensor-product weights
// [edges, paths*channels]).
//
//   C[M, N] = A[M, K] @ B[N, K]^T        (both operands K-major, C row-major, all fp32)
//
// Plain TF32 (10-bit mantissa) is too coarse for the 1e-5 eV/atom parity target, so every
// operand is split into a TF32-exact high part and a residual, x = hi + lo, and the product is
// accumulated as hi*hi + hi*lo + lo*hi in the FP32 TMEM accumulator (the dropped lo*lo term is
// ~2^-22 relative).  The weight operand B is split once on the host.  The activation operand A is split by the kernel
// right after its TMA load: one thread per row reads the row's 128 bytes (in the swizzled order the TMA engine wrote)
// and stores the high parts and the residuals to tensor memory, from where the tensor core takes its A operand
// (`tcgen05.mma` with A in TMEM, B from shared memory); a variant that keeps A in shared memory (split in place, residual
// in a second tile) remains selectable.
//
// One persistent CTA per SM walks its share of 128 x BN output tiles with specialised warps: a TMA
// producer fills a ring of {A, B_hi, B_lo} per 32-wide K step (four stages at BN = 128, six at BN = 64; three / four
// with A_lo in shared memory), four warps split A, one thread issues the tcgen05.mma instructions into one of two TMEM
// accumulators, and four epilogue warps drain the other accumulator (tcgen05.ld of their 32 lanes, 128-bit stores), so
// loads, splitting, tensor-core work and stores overlap.  The tensor core adds into its accumulator with truncation, an error that
// grows linearly with the number of accumulated instructions; long K loops are therefore cut
// into chunks of kChunk steps whose partial sums are drained from TMEM and added in FP32
// registers with round-to-nearest.  Every mbarrier wait is bounded: on expiry the CTA records an error code in
// global memory, stops waiting, drains and frees its TMEM, and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstring>
#include <cstdlib>

#include "../../include/tace_b200.h"
#include "kernels.h"

namespace tace {

namespace {

constexpr int kBM = 128;      // rows per tile = TMEM lanes
constexpr int kBK = 32;       // fp32 elements per K step = one 128-byte swizzle row
constexpr int kChunk = 8;     // K steps accumulated inside TMEM before draining into FP32 registers
constexpr int kTileABytes = kBM * kBK * 4;  // 16 KB
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred P1;\n mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n selp.b32 %0, 1, 0, P1;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the limit is hit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error, int code,
                                          uint32_t limit) {
  if (mbar_try_wait(bar, parity)) return !*abort_flag;  // the common case costs one probe
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return !*abort_flag;
    if ((it & 1023u) == 0u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(error, 0, code);
  return false;
}
// K-major operand tile with 128-byte rows and 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= (uint64_t)1 << 16;                          // leading byte offset (unused for this layout)
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// One linear problem of a launch: C[(atom, m), :] = A[(atom, m), 0:K] @ B[0:N, 0:K]^T (+ bias).
// Rows are (atom, component) pairs; the 3-D tensor map of A is {K, q, atoms} with box {32, q, R},
// R = 128 / q atoms per tile, so a tile's rows land in shared memory in (atom, m) order.
struct TcProblem {
  CUtensorMap tmA, tmBhi, tmBlo;  // B maps are 3-D {K, N, groups}
  float* C;
  const float* bias;     // [N] (per group) or nullptr
  long long c_s1, c_s2;  // atom stride / component stride of C rows (elements)
  long long bias_group_stride;
  int q, R, n_atoms, N, K;
  // per-species problems: atoms are sorted by species, group g owns atoms [group_ptr[g], group_ptr[g+1]) and
  // R-atom tiles [tile_ptr[g], tile_ptr[g+1]); both arrays live in device memory.  n_groups == 0: one group.
  int n_groups;
  const int* group_ptr;
  const int* tile_ptr;
  const int* atom_map;   // row of C for sorted atom a is atom_map[a]; nullptr: identity
  int accumulate;        // C += instead of C =
  int b_tiled;           // B maps are 4-D {32, N, K/32, groups} over K-tile-major weights
  int c_tma;             // plain row-major result (q = 1, no map, no accumulate): written by TMA stores through tmC
  CUtensorMap tmC;       // 2-D {N, rows}, box 32 x 32, 128-byte swizzle
};
constexpr int kTcMaxProblems = 4;
struct TcBatch {
  TcProblem p[kTcMaxProblems];
  int n_problems;
  int tile_start[kTcMaxProblems + 1];  // prefix sum of the problems' tile counts
  int* error;
  uint32_t spin_limit;   // polls per wait before a role gives up (kSpinLimit; smaller in the test mode)
  uint32_t extra_tx;     // test mode: bytes added to what the first load barrier expects, so that it never completes
};

// Warp roles (256 threads): warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-3 = operand
// splitters, warps 4-7 = epilogue (warp w owns the TMEM lanes 32 * (w % 4) .. + 31).
constexpr int kSplitThreads = 64;  // without TS: warps 2 and 3

// TS: the activation operand of the tensor-core instructions lives in tensor memory.  The splitters read the tile the TMA
// unit wrote and store its high part and residual to TMEM (one thread per row = TMEM lane), so a stage needs no room for
// them in shared memory: 48 KB instead of 64 KB at BN = 128, i.e. four K-steps in flight instead of three (six instead
// of four at BN = 64), and the tensor core reads only the weight operand from shared memory.  The ring's round trip, not any
// unit, is what bounds this kernel, so the number of stages in flight is its throughput.
template <int BN, bool TS>
struct TcSmem {
  static constexpr int kStages = TS ? (BN == 128 ? 4 : 6) : (BN == 128 ? 3 : 4);
  static constexpr int kTileBBytes = BN * kBK * 4;
  static constexpr int kStageBytes = (TS ? 1 : 2) * kTileABytes + 2 * kTileBBytes;
  static constexpr int kThreads = TS ? 320 : 256;        // TS: four splitter warps (2, 3, 8, 9), one per TMEM lane quarter
  static constexpr int kSplit = TS ? 128 : 64;           // splitter threads = arrivals on a `ready` barrier
  static constexpr int kTmemCols = TS ? 512 : 2 * BN;    // accumulators [0, 2 BN) | TS: per stage 32 columns high part, 32 residual
  static constexpr int kTmemA = 2 * BN;                  // first activation column (TS)
  static constexpr int kBarrierBytes = 256;
  // result staging for TMA stores: per epilogue warp two slabs of 32 rows x 32 columns (128-byte swizzled rows)
  static constexpr int kStoreBytes = 4 * 2 * 32 * 128;
  static constexpr int kTotal = kStages * kStageBytes + kStoreBytes + kBarrierBytes + 1024;  // + alignment slack
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y) : "memory");
}

struct TileInfo {
  int prob, atom0, atom_end, group, n0, num_k;
};
// tile_start: prefix sums of the problems' tile counts (in shared memory: grouped problems only know
// their tile count on the device)
template <int BN>
__device__ __forceinline__ TileInfo decode_tile(const TcBatch& b, const int* tile_start, int tile) {
  int pi = 0;
  while (pi + 1 < b.n_problems && tile >= tile_start[pi + 1]) ++pi;
  const TcProblem& P = b.p[pi];
  const int local = tile - tile_start[pi];
  const int tiles_n = P.N / BN;
  const int mt = local / tiles_n;
  TileInfo t;
  t.prob = pi;
  t.n0 = (local - mt * tiles_n) * BN;
  t.num_k = P.K / kBK;
  if (P.n_groups > 0) {
    int lo = 0, hi = P.n_groups;  // largest g with tile_ptr[g] <= mt
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (P.tile_ptr[mid] <= mt) lo = mid; else hi = mid;
    }
    t.group = lo;
    t.atom0 = P.group_ptr[lo] + (mt - P.tile_ptr[lo]) * P.R;
    t.atom_end = P.group_ptr[lo + 1];
  } else {
    t.group = 0;
    t.atom0 = mt * P.R;
    t.atom_end = P.n_atoms;
  }
  return t;
}

// ONE_CHUNK: every K loop of the launch fits one TMEM accumulation chunk, so the epilogue stores
// straight from the drained registers and needs no running sums.
template <int BN, bool ONE_CHUNK, bool TS>
__global__ void __launch_bounds__(TcSmem<BN, TS>::kThreads, 1) tc_gemm_kernel(const __grid_constant__ TcBatch batch) {
  using S = TcSmem<BN, TS>;
  constexpr int kStages = S::kStages;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128-byte-swizzled tiles need 1024-byte alignment
  unsigned char* base_ptr = smem_raw + (base - raw);
  const uint32_t store_base = base + kStages * S::kStageBytes;  // 1024-byte aligned: stage sizes are multiples of 1024
  const uint32_t bars = store_base + S::kStoreBytes;
  // barriers: raw[s] TMA landed | ready[s] operands split | empty[s] MMAs done reading | acc_full[a] | acc_empty[a]
  auto raw_bar = [&](int s) { return bars + 8u * s; };
  auto ready_bar = [&](int s) { return bars + 8u * (kStages + s); };
  auto empty_bar = [&](int s) { return bars + 8u * (2 * kStages + s); };
  auto acc_full = [&](int a) { return bars + 8u * (3 * kStages + a); };
  auto acc_empty = [&](int a) { return bars + 8u * (3 * kStages + 2 + a); };
  const uint32_t drain_bar = bars + 8u * (3 * kStages + 4);  // abort path only: issued tensor-core work has retired
  unsigned char* misc = base_ptr + kStages * S::kStageBytes + S::kStoreBytes + 8 * (3 * kStages + 5);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 8);
  int* tile_start = reinterpret_cast<int*>(misc + 16);  // [n_problems + 1]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {  // `ready` takes one arrival per splitter warp
    for (int s = 0; s < kStages; ++s) { mbar_init(raw_bar(s), 1); mbar_init(ready_bar(s), S::kSplit / 32); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 128); }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    int acc = 0;
    for (int i = 0; i < batch.n_problems; ++i) {
      const TcProblem& P = batch.p[i];
      tile_start[i] = acc;
      const int tiles_m = P.n_groups > 0 ? P.tile_ptr[P.n_groups] : (P.n_atoms + P.R - 1) / P.R;
      acc += tiles_m * (P.N / BN);
    }
    for (int i = batch.n_problems; i <= kTcMaxProblems; ++i) tile_start[i] = acc;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // two accumulators of BN fp32 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(S::kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int n_tiles = tile_start[batch.n_problems];
  // instruction descriptor: D = F32, A = B = TF32, both K-major, N = BN, M = 128
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  auto stage_a = [&](int s) { return base + s * S::kStageBytes; };
  constexpr int kBOff = (TS ? 1 : 2) * kTileABytes;  // weights follow the activation tile (and, without TS, its residual)
  auto stage_alo = [&](int s) { return base + s * S::kStageBytes + kTileABytes; };  // not TS
  auto stage_bhi = [&](int s) { return base + s * S::kStageBytes + kBOff; };
  auto stage_blo = [&](int s) { return base + s * S::kStageBytes + kBOff + S::kTileBBytes; };

  if (warp == 0) {
    // ---- TMA producer
    if (lane == 0) {
      int step = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const TileInfo t = decode_tile<BN>(batch, tile_start, tile);
        const TcProblem& P = batch.p[t.prob];
        const uint32_t a_bytes = (uint32_t)P.R * P.q * kBK * 4;
        for (int ks = 0; ks < t.num_k; ++ks, ++step) {
          const int s = step % kStages, ph = (step / kStages) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, batch.error, 1, batch.spin_limit)) { ok = false; break; }
          mbar_expect_tx(raw_bar(s), a_bytes + 2 * S::kTileBBytes + batch.extra_tx);
          tma_load_3d(stage_a(s), &P.tmA, raw_bar(s), ks * kBK, 0, t.atom0);
          if (P.b_tiled) {  // weights stored K-tile-major: one contiguous block per (k-step, n-tile)
            tma_load_4d(stage_bhi(s), &P.tmBhi, raw_bar(s), 0, t.n0, ks, t.group);
            tma_load_4d(stage_blo(s), &P.tmBlo, raw_bar(s), 0, t.n0, ks, t.group);
          } else {
            tma_load_3d(stage_bhi(s), &P.tmBhi, raw_bar(s), ks * kBK, t.n0, t.group);
            tma_load_3d(stage_blo(s), &P.tmBlo, raw_bar(s), ks * kBK, t.n0, t.group);
          }
        }
      }
      if (*abort_flag) {  // loads already issued must land before the CTA exits
        for (int j = step > kStages ? step - kStages : 0; j < step; ++j) {
          const int s = j % kStages, ph = (j / kStages) & 1;
          for (uint32_t it = 0; it < batch.spin_limit; ++it)
            if (mbar_try_wait(raw_bar(s), ph)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      int chunk = 0;
      bool ok = true;
      // This one thread issues every tensor-core instruction of the SM, and its own instruction stream is part of what
      // the ring waits for: descriptors are built once (only their 14-bit start-address field, in 16-byte units, changes
      // from stage to stage and from one 8-wide K slice to the next, so the later ones are sums), and the stage index and
      // phase are counted instead of divided.
      const uint64_t dA0 = umma_desc(stage_a(0)), dAl0 = umma_desc(stage_alo(0));
      const uint64_t dB0 = umma_desc(stage_bhi(0)), dBl0 = umma_desc(stage_blo(0));
      int s = 0, ph = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const TileInfo t = decode_tile<BN>(batch, tile_start, tile);
        for (int ks = 0; ks < t.num_k; ++ks, ph ^= (s == kStages - 1), s = (s == kStages - 1) ? 0 : s + 1) {
          const int a = chunk & 1;
          const bool chunk_begin = (ks % kChunk) == 0;
          const bool chunk_end = (ks % kChunk) == kChunk - 1 || ks == t.num_k - 1;
          if (chunk_begin && !mbar_wait(acc_empty(a), ((chunk >> 1) & 1) ^ 1, abort_flag, batch.error, 4, batch.spin_limit)) { ok = false; break; }
          if (!mbar_wait(ready_bar(s), ph, abort_flag, batch.error, 2, batch.spin_limit)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t d = tmem_base + a * BN;
          const uint64_t stage_off = (uint64_t)((uint32_t)(s * S::kStageBytes) >> 4);
#pragma unroll
          for (int k8 = 0; k8 < kBK / 8; ++k8) {
            const uint64_t off = stage_off + (uint64_t)(k8 * 2);  // 8 fp32 = 32 bytes along K inside the swizzled row
            const uint64_t db = dB0 + off, dbl = dBl0 + off;
            if constexpr (TS) {  // activations: 8 TMEM columns per slice, high part at +0, residual at +32 of the stage
              const uint32_t ta = tmem_base + (uint32_t)(S::kTmemA + s * 64 + k8 * 8);
              umma_tf32_ts(d, ta, db, idesc, (!chunk_begin || k8 > 0) ? 1u : 0u);
              umma_tf32_ts(d, ta, dbl, idesc, 1u);
              umma_tf32_ts(d, ta + 32, db, idesc, 1u);
            } else {
              const uint64_t da = dA0 + off, dal = dAl0 + off;
              umma_tf32(d, da, db, idesc, (!chunk_begin || k8 > 0) ? 1u : 0u);
              umma_tf32(d, da, dbl, idesc, 1u);
              umma_tf32(d, dal, db, idesc, 1u);
            }
          }
          umma_commit(empty_bar(s));  // ring slot reusable once these MMAs have read it
          if (chunk_end) { umma_commit(acc_full(a)); ++chunk; }  // partial sum of this chunk complete
        }
      }
      if (*abort_flag) {  // tensor-core work already issued must retire before the tensor memory is given back
        umma_commit(drain_bar);
        for (uint32_t it = 0; it < batch.spin_limit; ++it)
          if (mbar_try_wait(drain_bar, 0)) break;
      }
    }
  } else if (warp < 4 || (TS && warp >= 8)) {
    // ---- operand splitters: A = hi + lo with hi exact in TF32
    const int t64 = tid - 64;
    int step = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const TileInfo t = decode_tile<BN>(batch, tile_start, tile);
      for (int ks = 0; ks < t.num_k; ++ks, ++step) {
        const int s = step % kStages, ph = (step / kStages) & 1;
        if (!mbar_wait(raw_bar(s), ph, abort_flag, batch.error, 3, batch.spin_limit)) { ok = false; break; }
        if constexpr (TS) {
          // one thread per row (= TMEM lane): the row's eight 16-byte pieces sit at positions j ^ (row & 7) of its 128 bytes
          // (the swizzle the TMA unit wrote); high parts go to 32 TMEM columns of the stage, residuals to the next 32
          const int row = (warp & 3) * 32 + lane;
          const float4* arow = reinterpret_cast<const float4*>(base_ptr + s * S::kStageBytes + row * 128);
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = arow[j ^ (row & 7)];
            const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t h = __float_as_uint(x[q]) & 0xFFFFE000u;
              hi[4 * j + q] = h;
              lo[4 * j + q] = __float_as_uint(x[q] - __uint_as_float(h));
            }
          }
          const uint32_t ta = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(S::kTmemA + s * 64);
          tmem_st32(ta, hi);
          tmem_st32(ta + 32, lo);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(ready_bar(s));
          continue;
        }
        float4* a = reinterpret_cast<float4*>(base_ptr + s * S::kStageBytes);
        float4* alo = reinterpret_cast<float4*>(base_ptr + s * S::kStageBytes + kTileABytes);
        // every load of the tile before its first store: the stores go to the buffer the loads come from, so the compiler
        // must keep their order, and sixteen dependent load -> store rounds would put their latencies end to end on the
        // critical path of the operand ring
        constexpr int kPer = kTileABytes / 16 / kSplitThreads;
        float4 v[kPer];
#pragma unroll
        for (int j = 0; j < kPer; ++j) v[j] = a[t64 + j * kSplitThreads];
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          const int idx = t64 + j * kSplitThreads;
          float4 h, l;
          h.x = __uint_as_float(__float_as_uint(v[j].x) & 0xFFFFE000u); l.x = v[j].x - h.x;
          h.y = __uint_as_float(__float_as_uint(v[j].y) & 0xFFFFE000u); l.y = v[j].y - h.y;
          h.z = __uint_as_float(__float_as_uint(v[j].z) & 0xFFFFE000u); l.z = v[j].z - h.z;
          h.w = __uint_as_float(__float_as_uint(v[j].w) & 0xFFFFE000u); l.w = v[j].w - h.w;
          a[idx] = h;
          alo[idx] = l;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_bar(s));
      }
    }
  } else {
    // ---- epilogue: drain each chunk's partial sum from TMEM, add in FP32 registers, store at tile end
    const int ew = warp & 3;  // a warp may only touch TMEM lanes 32 * (warp % 4) .. + 31
    float accr[ONE_CHUNK ? 1 : BN];
    int chunk = 0, slab = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const TileInfo t = decode_tile<BN>(batch, tile_start, tile);
      const TcProblem& P = batch.p[t.prob];
      const int r = ew * 32 + lane;
      const int al = r / P.q, m = r - al * P.q;
      const bool valid = r < P.R * P.q && t.atom0 + al < t.atom_end;
      long long atom = t.atom0 + al;
      if (valid && P.atom_map) atom = P.atom_map[atom];
      float* dst = P.C + atom * P.c_s1 + (long long)m * P.c_s2 + t.n0;
      const float* bias = P.bias ? P.bias + t.group * P.bias_group_stride + t.n0 : nullptr;
      const bool accumulate = P.accumulate != 0;
      const int n_chunks = (t.num_k + kChunk - 1) / kChunk;
      for (int cin = 0; cin < n_chunks; ++cin, ++chunk) {
        const int a = chunk & 1;
        if (!mbar_wait(acc_full(a), (chunk >> 1) & 1, abort_flag, batch.error, 5, batch.spin_limit)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t rr[32];
          tmem_ld32(tmem_base + ((uint32_t)(ew * 32) << 16) + a * BN + c * 32, rr);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if constexpr (ONE_CHUNK) {
            if (P.c_tma) {
              // stage the warp's 32 x 32 slab in shared memory (16-byte chunk j of row r at chunk j ^ (r & 7), the
              // 128-byte swizzle of the tensor map) and let the TMA unit write whole 128-byte rows; rows past the
              // end of the tensor are clipped by the hardware
              const uint32_t buf = store_base + (uint32_t)((ew * 2 + (slab & 1)) * 32 * 128);
              if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // slab - 2 has left this buffer
              __syncwarp();
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                float4 v = make_float4(__uint_as_float(rr[4 * q4]), __uint_as_float(rr[4 * q4 + 1]), __uint_as_float(rr[4 * q4 + 2]),
                                       __uint_as_float(rr[4 * q4 + 3]));
                if (bias) {
                  const float4 bv = *reinterpret_cast<const float4*>(bias + c * 32 + 4 * q4);
                  v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
                }
                const uint32_t addr = buf + (uint32_t)(lane * 128 + ((q4 ^ (lane & 7)) << 4));
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
              }
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> TMA reads
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&P.tmC, buf, t.n0 + c * 32, t.atom0 + ew * 32);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              }
              ++slab;
            } else if (valid) {
              // all loads of a slab before its first store: a load that follows a store to the same 128-byte line
              // waits for that store to be acknowledged by L2, which would serialise the row
              float4 v[8];
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4)
                v[q4] = make_float4(__uint_as_float(rr[4 * q4]), __uint_as_float(rr[4 * q4 + 1]), __uint_as_float(rr[4 * q4 + 2]),
                                    __uint_as_float(rr[4 * q4 + 3]));
              if (bias) {
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) {
                  const float4 bv = *reinterpret_cast<const float4*>(bias + c * 32 + 4 * q4);
                  v[q4].x += bv.x; v[q4].y += bv.y; v[q4].z += bv.z; v[q4].w += bv.w;
                }
              }
              if (accumulate) {
                float4 ov[8];
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) ov[q4] = *reinterpret_cast<const float4*>(dst + c * 32 + 4 * q4);
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) { v[q4].x += ov[q4].x; v[q4].y += ov[q4].y; v[q4].z += ov[q4].z; v[q4].w += ov[q4].w; }
              }
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) *reinterpret_cast<float4*>(dst + c * 32 + 4 * q4) = v[q4];
            }
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) accr[c * 32 + q] = cin == 0 ? __uint_as_float(rr[q]) : accr[c * 32 + q] + __uint_as_float(rr[q]);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(acc_empty(a));  // the issuer may overwrite this accumulator
        if constexpr (!ONE_CHUNK) {
          if (cin == n_chunks - 1 && valid) {
            if (accumulate) {  // every load of the row before its first store (see above)
#pragma unroll
              for (int q4 = 0; q4 < BN / 4; ++q4) {
                const float4 ov = *reinterpret_cast<const float4*>(dst + 4 * q4);
                accr[4 * q4] += ov.x; accr[4 * q4 + 1] += ov.y; accr[4 * q4 + 2] += ov.z; accr[4 * q4 + 3] += ov.w;
              }
            }
            if (bias) {
#pragma unroll
              for (int q4 = 0; q4 < BN / 4; ++q4) {
                const float4 bv = *reinterpret_cast<const float4*>(bias + 4 * q4);
                accr[4 * q4] += bv.x; accr[4 * q4 + 1] += bv.y; accr[4 * q4 + 2] += bv.z; accr[4 * q4 + 3] += bv.w;
              }
            }
#pragma unroll
            for (int q4 = 0; q4 < BN / 4; ++q4)
              *reinterpret_cast<float4*>(dst + 4 * q4) = make_float4(accr[4 * q4], accr[4 * q4 + 1], accr[4 * q4 + 2], accr[4 * q4 + 3]);
          }
        }
      }
    }
  }
  if (warp >= 4 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // TMA stores of this warp are complete
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::kTmemCols));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 3-D fp32 weight tensor [groups][N][K]; box = [1][box_rows][32], 128-byte swizzle.
bool make_map_b(CUtensorMap* map, const float* ptr, int groups, long long N, long long K, long long group_stride, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)N, (cuuint64_t)groups};
  const cuuint64_t strides[2] = {(cuuint64_t)K * sizeof(float), (cuuint64_t)(groups > 1 ? group_stride : N * K) * sizeof(float)};
  const cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// The same weights stored K-tile-major, [groups][K/32][N][32]: the 128-byte rows of one (k-step, n-tile) operand block are
// adjacent in memory, so a block that is read once from DRAM (per-species weights) streams as whole pages.
bool make_map_b_tiled(CUtensorMap* map, const float* ptr, int groups, long long N, long long K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)kBK, (cuuint64_t)N, (cuuint64_t)(K / kBK), (cuuint64_t)groups};
  const cuuint64_t strides[3] = {(cuuint64_t)kBK * sizeof(float), (cuuint64_t)N * kBK * sizeof(float), (cuuint64_t)N * K * sizeof(float)};
  const cuuint32_t box[4] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// 3-D fp32 tensor [atoms][q][K]; box = [R atoms][q][32], 128-byte swizzle.
bool make_map_3d(CUtensorMap* map, const float* ptr, long long atoms, int q, long long K, long long atom_stride,
                 long long comp_stride, int R) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)q, (cuuint64_t)atoms};
  const cuuint64_t strides[2] = {(cuuint64_t)(q == 1 ? atom_stride : comp_stride) * sizeof(float),
                                 (cuuint64_t)atom_stride * sizeof(float)};
  const cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)q, (cuuint32_t)R};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D fp32 result [rows][N] with row stride ldc; box = 32 rows x 32 columns, 128-byte swizzle.
bool make_map_c(CUtensorMap* map, float* ptr, long long rows, long long N, long long ldc) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ldc * sizeof(float)};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Function attributes and the SM count belong to a device, not to the process: one slot per device ordinal.
constexpr int kMaxDevices = 64;

template <int BN, bool ONE_CHUNK, bool TS>
cudaError_t launch_tc_v(const TcBatch& b, int dev, int sms, cudaStream_t s) {
  static bool configured[kMaxDevices] = {};
  using S = TcSmem<BN, TS>;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tc_gemm_kernel<BN, ONE_CHUNK, TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int tiles = b.tile_start[b.n_problems];  // upper bound for per-species problems
  const int grid = tiles < sms ? tiles : sms;
  tc_gemm_kernel<BN, ONE_CHUNK, TS><<<grid, S::kThreads, S::kTotal, s>>>(b);
  return cudaGetLastError();
}
template <int BN, bool ONE_CHUNK>
cudaError_t launch_tc(const TcBatch& b, int dev, int sms, cudaStream_t s) {
  // TACE_B200_GEMM_TMEM_OPERAND=0 selects the variant with both operands in shared memory (three / four stages)
  static const bool ts = [] { const char* e = getenv("TACE_B200_GEMM_TMEM_OPERAND"); return !(e && e[0] == '0'); }();
  return ts ? launch_tc_v<BN, ONE_CHUNK, true>(b, dev, sms, s) : launch_tc_v<BN, ONE_CHUNK, false>(b, dev, sms, s);
}

}  // namespace

// Test mode of the bounded waits (tace_tc_gemm_set_test_mode): a short poll limit, and a byte count added to what the
// load barriers expect so that they never complete; both 0 in normal operation.
static uint32_t g_test_spin_limit = 0, g_test_extra_tx = 0;
void tc_gemm_set_test_mode(uint32_t spin_limit, uint32_t extra_tx) { g_test_spin_limit = spin_limit; g_test_extra_tx = extra_tx; }

bool tc_linear_supported(int N, int K) { return N % 64 == 0 && K % kBK == 0; }

cudaError_t launch_tc_linear(const TcLinearProblem* probs, int n_problems, int* error_flag, cudaStream_t s) {
  if (n_problems <= 0) return cudaSuccess;
  if (n_problems > kTcMaxProblems || !error_flag) return cudaErrorInvalidValue;
  static int sms_of[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidValue;
  if (!sms_of[dev] && cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return cudaErrorInvalidValue;
  const int sms = sms_of[dev];
  bool all128 = true, one = true;
  for (int i = 0; i < n_problems; ++i) {
    const TcLinearProblem& h = probs[i];
    if (!tc_linear_supported(h.N, h.K) || h.q < 1 || h.q > 128 || (h.a_atom_stride & 3) || (h.a_comp_stride & 3) || (h.c_s1 & 3) ||
        (h.c_s2 & 3))
      return cudaErrorInvalidValue;
    all128 = all128 && (h.N % 128 == 0);
    one = one && (h.K / kBK <= kChunk);
  }
  const int bn = all128 ? 128 : 64;
  TcBatch b;
  memset(&b, 0, sizeof(b));
  b.n_problems = 0;
  b.error = error_flag;
  b.spin_limit = g_test_spin_limit ? g_test_spin_limit : kSpinLimit;
  b.extra_tx = g_test_extra_tx;
  int tiles = 0;
  for (int i = 0; i < n_problems; ++i) {
    const TcLinearProblem& h = probs[i];
    if (h.n_atoms <= 0) continue;
    TcProblem& P = b.p[b.n_problems];
    P.q = h.q; P.R = kBM / h.q; P.n_atoms = (int)h.n_atoms; P.N = h.N; P.K = h.K;
    P.C = h.C; P.bias = h.bias; P.c_s1 = h.c_s1; P.c_s2 = h.c_s2; P.bias_group_stride = h.bias_group_stride;
    P.n_groups = h.n_groups; P.group_ptr = h.group_ptr; P.tile_ptr = h.tile_ptr; P.atom_map = h.atom_map;
    P.accumulate = h.accumulate;
    const int groups = h.n_groups > 0 ? h.n_groups : 1;
    if (h.n_groups > 0 && (!h.group_ptr || !h.tile_ptr)) return cudaErrorInvalidValue;
    P.b_tiled = h.b_tiled;
    if (h.b_tiled && groups > 1 && h.b_group_stride != (long long)h.N * h.K) return cudaErrorInvalidValue;
    if (!make_map_3d(&P.tmA, h.A, h.n_atoms, h.q, h.K, h.a_atom_stride, h.a_comp_stride, P.R)) return cudaErrorInvalidValue;
    if (h.b_tiled ? (!make_map_b_tiled(&P.tmBhi, h.Bhi, groups, h.N, h.K, bn) || !make_map_b_tiled(&P.tmBlo, h.Blo, groups, h.N, h.K, bn))
                  : (!make_map_b(&P.tmBhi, h.Bhi, groups, h.N, h.K, h.b_group_stride, bn) ||
                     !make_map_b(&P.tmBlo, h.Blo, groups, h.N, h.K, h.b_group_stride, bn)))
      return cudaErrorInvalidValue;
    // large plain results (the per-edge weights of the radial MLP) leave through TMA stores
    P.c_tma = 0;
    if (one && h.q == 1 && h.n_groups == 0 && !h.atom_map && !h.accumulate && (reinterpret_cast<uintptr_t>(h.C) & 15) == 0) {
      if (!make_map_c(&P.tmC, h.C, h.n_atoms, h.N, h.c_s1)) return cudaErrorInvalidValue;
      P.c_tma = 1;
    }
    b.tile_start[b.n_problems] = tiles;
    tiles += (int)((h.n_atoms + P.R - 1) / P.R + h.n_groups) * (h.N / bn);
    ++b.n_problems;
  }
  for (int i = b.n_problems; i <= kTcMaxProblems; ++i) b.tile_start[i] = tiles;
  if (tiles == 0) return cudaSuccess;
  if (bn == 128) return one ? launch_tc<128, true>(b, dev, sms, s) : launch_tc<128, false>(b, dev, sms, s);
  return one ? launch_tc<64, true>(b, dev, sms, s) : launch_tc<64, false>(b, dev, sms, s);
}

cudaError_t launch_tc_gemm(const float* A, long long lda, const float* Bhi, const float* Blo, float* C, long long ldc, int M,
                           int N, int K, int* error_flag, cudaStream_t s, const float* bias) {
  if (M <= 0) return cudaSuccess;
  TcLinearProblem h;
  memset(&h, 0, sizeof(h));
  h.A = A; h.a_atom_stride = lda; h.a_comp_stride = lda; h.q = 1; h.n_atoms = M; h.K = K;
  h.Bhi = Bhi; h.Blo = Blo; h.N = N; h.C = C; h.c_s1 = ldc; h.c_s2 = 0; h.bias = bias;
  return launch_tc_linear(&h, 1, error_flag, s);
}

}  // namespace tace

extern "C" int tace_tc_gemm_f32(const float* A, int64_t lda, const float* B_hi, const float* B_lo, float* C, int64_t ldc,
                                int32_t M, int32_t N, int32_t K, int32_t* error_flag, tace_stream_t stream) {
  if (!A || !B_hi || !B_lo || !C) return TACE_ERR_INVALID_ARGUMENT;
  cudaError_t e = tace::launch_tc_gemm(A, lda, B_hi, B_lo, C, ldc, M, N, K, error_flag, static_cast<cudaStream_t>(stream), nullptr);
  if (e == cudaErrorInvalidValue) return TACE_ERR_INVALID_ARGUMENT;
  return e == cudaSuccess ? TACE_OK : TACE_ERR_CUDA;
}

extern "C" int tace_tc_gemm_set_test_mode(uint32_t spin_limit, uint32_t extra_expected_bytes) {
  tace::tc_gemm_set_test_mode(spin_limit, extra_expected_bytes);
  return TACE_OK;
}
