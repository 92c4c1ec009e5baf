// B200 (sm_100a) pi0.5 action-chunk engine: the whole chunk (time MLP + adaRMS modulations, then
// n_steps Euler steps x n_layers Gemma-300M expert layers) as ONE persistent kernel, plus the C ABI.
//
// Semantics follow the reference's eager definition of the chunk (reference/pi05.py:218-309) and the rounding
// schedule its own megakernel uses (mk/pi05_mk.cu:2609-2643 RoPE, 2797-2836 attention, 1301-1327 residual,
// 1453-1475 step tail).  The structure is new:
//
//   * CTAs have fixed roles.  "GEMM CTAs" stream BF16 weights with TMA into a deep shared-memory ring and run
//     tcgen05 MMAs (weights on the M=128 side, the 50 tokens padded to N=64, FP32 accumulators in TMEM).  Their
//     weight producer never waits for activations, so HBM keeps streaming across stage, layer and step
//     boundaries.  "Row CTAs" run attention (warp MMA, online softmax over 64-key chunks) and the per-token
//     row operations (gated residual, adaRMS, Euler step, action projections).
//   * Stages are ordered by device-scope counters (release add / acquire poll) that only the producers of a
//     stage bump and only its consumers poll; there is no grid-wide barrier inside the layer loop.
//   * Every wait is bounded.  A wait that gives up writes a status word, every other wait sees it and the
//     kernel drains and exits; the host reads the word through pi05_status().
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/pi05_b200.h"
#include "ptx_sm100.cuh"

#include "pi05_common.cuh"
using namespace pi05;

// Four builds of the same device code (see pi05_chunk_kernel.cuh): the production kernel for one observation, the
// batched kernels with one or two observations per MMA, and the traced kernel (one observation per MMA) for
// callers that ask for stamps or debug controls.
#ifndef PI05_QF_KEPT
#define PI05_QF_KEPT 8
#endif
namespace k_plain {
#define PI05_TRACE 0
#define PI05_BATCHED 0
#define PI05_GN 1
#define PI05_TP 0
#include "pi05_chunk_kernel.cuh"
#undef PI05_TRACE
#undef PI05_BATCHED
#undef PI05_GN
#undef PI05_TP
}  // namespace k_plain
namespace k_batched {
#define PI05_TRACE 0
#define PI05_BATCHED 1
#define PI05_GN 1
#define PI05_TP 0
#include "pi05_chunk_kernel.cuh"
#undef PI05_TRACE
#undef PI05_BATCHED
#undef PI05_GN
#undef PI05_TP
}  // namespace k_batched
namespace k_pairs {
#define PI05_TRACE 0
#define PI05_BATCHED 1
#define PI05_GN 2
#define PI05_TP 0
#include "pi05_chunk_kernel.cuh"
#undef PI05_TRACE
#undef PI05_BATCHED
#undef PI05_GN
#undef PI05_TP
}  // namespace k_pairs
namespace k_tp {
#define PI05_TRACE 0
#define PI05_BATCHED 0
#define PI05_GN 1
#define PI05_TP 1
#include "pi05_chunk_kernel.cuh"
#undef PI05_TRACE
#undef PI05_BATCHED
#undef PI05_GN
#undef PI05_TP
}  // namespace k_tp
namespace k_traced {
#define PI05_TRACE 1
#define PI05_BATCHED 1
#define PI05_GN 1
#define PI05_TP 0
#include "pi05_chunk_kernel.cuh"
#undef PI05_TRACE
#undef PI05_BATCHED
#undef PI05_GN
#undef PI05_TP
}  // namespace k_traced

#ifndef PI05_PAIRS_FROM
// Batch sizes from this one on run two observations per MMA.  Beyond the largest batch: with the two-stream schedule
// one observation per MMA is faster at every batch size measured (B = 16: 18.8 against 19.4 ms per launch), so pairs
// only run when the tuning variable PI05_OBS_PER_MMA asks for them.
#define PI05_PAIRS_FROM 1000
#endif
namespace {
const void* const kAllKernels[] = {(const void*)k_plain::pi05_chunk_kernel, (const void*)k_batched::pi05_chunk_kernel,
                                   (const void*)k_pairs::pi05_chunk_kernel,
                                   (const void*)k_traced::pi05_chunk_kernel, (const void*)k_tp::pi05_chunk_kernel};
}  // namespace

// =========================================================================================== host side
namespace {
struct Region { const char* name; size_t off, bytes; };
}  // namespace


struct pi05_engine {
  int device = 0;
  int sms = 0;
  int grid = 0;
  int n_gemm = 0;
  int max_prefix = 0;
  int prefix = 0;
  int max_batch = 1;
  int batch = 1;
  int row_groups = 1;
  int key_groups = 1;
  int pages_per_obs = 1, page_tokens = 1;
  bool clustered = false;        // launched as clusters of two CTAs: consecutive blocks share a TPC
  bool bound = false;
  const void* inputs[PI05_NUM_INPUTS] = {};
  void* actions = nullptr;
  uint8_t* ws = nullptr;
  size_t ws_bytes = 0;
  std::vector<Region> regions;
  std::vector<Unit> sched;       // [grid][MAX_UNITS]
  std::vector<int> sched_n;
  int n_units[4] = {0, 0, 0, 0};
  TMaps maps;
  int tp_rank = 0, tp_size = 1;  // tensor parallel: this engine's share of one observation
  unsigned int tp_base = 0;      // arrivals per exchange counter consumed by earlier launches of this binding
  float* tp_peer_recv[MAX_TP] = {};
  unsigned int* tp_peer_flags[MAX_TP] = {};
  void* tp_opened[MAX_TP] = {};  // base addresses opened with cudaIpcOpenMemHandle (closed at destroy)
  pi05_tuning tune;              // every tuning setting (pi05_tune); defaults from pi05_tuning_defaults
  int gn = 1;                    // observations per MMA of the bound batch
  int stream_split = 0;          // groups in the first stream (0: one stream)
  int max_stage = 0x7fffffff;
  int drop_event = -1;
  long long wait_limit = 4000000000ll;    // ~2 s of SM clocks
  unsigned long long launches = 0;
  cudaEvent_t done = nullptr;    // recorded after this handle's last launch, on that launch's stream
  cudaStream_t side = nullptr;   // non-blocking stream for the few bytes pi05_status moves (never the legacy default stream,
                                 // which would serialise against every other stream of the GPU)
  bool in_flight = false;        // a launch has been issued since the last pi05_status
  bool can_cluster = false;      // the device takes the whole grid as clusters of two
  std::string config;
  std::string last_error;
};

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    ok = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

int fail_cuda(pi05_engine* h, const char* what, cudaError_t e) {
  h->last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return PI05_ERR_CUDA;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

void build_layout(pi05_engine* h) {
  size_t off = 0;
  auto add = [&](const char* name, size_t bytes) {
    h->regions.push_back({name, off, bytes});
    off = align_up(off + bytes, 256);
  };
  const size_t B = (size_t)h->max_batch;      // per-observation buffers: observation b at b * (size / B)
  add("ctrl", CTRL_BYTES);
  add("temb", (size_t)NS * W * 4);
  add("hid", (size_t)NS * W * 4);
  add("cond", (size_t)NS * W * 4);
  add("mod", (size_t)NS * NNORM * MODW * 4);
  add("rope", B * T * (HD / 2) * 4);
  add("rope2", B * T * (HD / 2) * 4);
  add("x", B * T * ADIM * 4);
  add("h", B * T * W * 2);
  add("an_attn", B * AN_COPIES * T * W * 2);
  add("an_ffn", B * AN_COPIES * T * W * 2);
  add("qkv_acc", B * T * QKVW * 4);
  add("k", B * T * HD * 2);
  add("v", B * T * HD * 2);
  add("attn", B * T * QD * 2);
  add("o_acc", B * T * W * 4);
  add("d_acc", B * T * W * 4);
  add("act", B * T * FF * 2);
  add("att_part", (size_t)(MAX_KEY_GROUPS - 1) * NROW_CTAS * ATT_PART_FLOATS * 4);
  if (h->tp_size > 1) {          // what the peers write into (see pi05_common.cuh)
    add("tp_recv", (size_t)2 * h->tp_size * TP_SLOT_FLOATS * 4);
    add("tp_flags", (size_t)2 * NROW_CTAS * TP_FLAG_STRIDE * 4);
  }
  add("page_table", (size_t)h->max_batch * ((h->max_prefix + 63) / 64) * sizeof(int));
  add("sched", (size_t)h->grid * MAX_UNITS * sizeof(Unit));
  add("sched_n", (size_t)h->grid * sizeof(int));
  h->ws_bytes = off;
}

const Region* find_region(const pi05_engine* h, const char* name) {
  for (const Region& r : h->regions)
    if (strcmp(r.name, name) == 0) return &r;
  return nullptr;
}

template <typename Tp>
Tp* region_ptr(const pi05_engine* h, const char* name) {
  return reinterpret_cast<Tp*>(h->ws + find_region(h, name)->off);
}

// Static work schedule: which CTA runs which 128-row weight tile over which range of 128-wide K stages.
// One observation (the latency schedule, every entry serves "all groups" = the one there is):
//   gate/up: 64 tiles (64 gate rows + the matching 64 up rows), full K, one per CTA 0..63
//   QKV:     16 q tiles x 4 K parts on the gate/up CTAs, 4 k / v tiles x full K on CTAs 64..67
//   O, down: 8 row tiles each, K split in contiguous runs over all GEMM CTAs (partial sums meet in L2)
// Tensor parallel (rank r of n): the same lists restricted to this rank's share - query heads 8 r / n .. (wq rows, and
// the matching K range of wo), MLP columns 4096 r / n .. (wg / wu rows, K range of wd) - with the single KV head's k / v
// tiles on every rank (reference/pi05.py:254-265 and 268-279 are what gets cut).
bool schedule_one(pi05_engine* h, std::vector<std::vector<Unit>>& per) {
  const int ng = h->n_gemm;
  if (h->tp_size > 1) {
    const int n = h->tp_size, r = h->tp_rank;
    for (int u = 0; u < NKVTILES; ++u) per[64 + u].push_back(Unit{G_QKV, 16 + u, 0, W / KSTAGE});
    const int qt = 16 / n, gt = 64 / n;                       // q tiles and gate/up tiles of this rank
    for (int u = 0; u < qt * 4; ++u) per[u].push_back(Unit{G_QKV, r * qt + u / 4, (u % 4) * 2, 2});
    const int per_tile = ng / (W / 128);
    auto split = [&](int gemm, int tiles, int stage0, int stages) {
      for (int t = 0; t < tiles; ++t)
        for (int j = 0; j < per_tile; ++j) {
          const int a0 = stages * j / per_tile, a1 = stages * (j + 1) / per_tile;
          if (a1 > a0) per[t * per_tile + j].push_back(Unit{gemm, t, stage0 + a0, a1 - a0});
        }
    };
    split(G_O, W / 128, r * (QD / KSTAGE / n), QD / KSTAGE / n);
    for (int u = 0; u < gt; ++u) per[u].push_back(Unit{G_GU, r * gt + u, 0, W / KSTAGE});
    split(G_DOWN, W / 128, r * (FF / KSTAGE / n), FF / KSTAGE / n);
    return true;
  }
  // QKV: the 4 k / v tiles over the full K on CTAs 64..67 (BF16 keys / values with RoPE straight from the epilogue);
  // the 16 q tiles in 4 two-stage K parts, one on each gate/up CTA (FP32 sums, finished by attention)
  for (int u = 0; u < NKVTILES; ++u) per[64 + u].push_back(Unit{G_QKV, 16 + u, 0, W / KSTAGE});
  for (int u = 0; u < 64; ++u) per[u].push_back(Unit{G_QKV, u / 4, (u % 4) * 2, 2});
  // every row tile gets the same number of CTAs and no CTA straddles two tiles (one unit, one epilogue per CTA)
  const int per_tile = ng / (W / 128);
  auto split = [&](int gemm, int tiles, int stages_per_tile) {
    for (int t = 0; t < tiles; ++t)
      for (int j = 0; j < per_tile; ++j) {
        const int a0 = stages_per_tile * j / per_tile, a1 = stages_per_tile * (j + 1) / per_tile;
        if (a1 > a0) per[t * per_tile + j].push_back(Unit{gemm, t, a0, a1 - a0});
      }
  };
  split(G_O, W / 128, QD / KSTAGE);
  for (int u = 0; u < 64; ++u) per[u].push_back(Unit{G_GU, u, 0, W / KSTAGE});
  split(G_DOWN, W / 128, FF / KSTAGE);
  return true;
}

// Several observations (the throughput schedule): every entry names the group of observations it serves, and the
// entries of each phase (k / v and q, O, gate/up, down) are dealt over ALL GEMM CTAs by load, so that no phase is
// left to a few CTAs while the others wait (with the latency schedule the k / v tiles of every group would queue on
// four CTAs and the gate/up tiles on 64).  Every CTA's list is in (phase, group) order, the same global order for
// all, so whatever an entry waits for is produced by entries that come earlier in that order, or by row CTAs.
// The K splits get coarser as the number of groups grows (about two entries per CTA and phase): fewer, longer
// units mean fewer epilogues and atomics.
bool schedule_groups(pi05_engine* h, std::vector<std::vector<Unit>>& per, int ngroups) {
  const int ng = h->n_gemm;
  std::vector<int> total(ng, 0);
  // deal the entries of one phase for groups [g0, g1) over the CTAs, least loaded (in this phase, then overall) first
  auto deal = [&](int gemm, int ntiles, int tile0, int stages, int parts, std::vector<int>& load, int g0, int g1, int lag) {
    for (int g = g0; g < g1; ++g)
      for (int t = 0; t < ntiles; ++t)
        for (int j = 0; j < parts; ++j) {
          const int a0 = stages * j / parts, a1 = stages * (j + 1) / parts;
          if (a1 <= a0) continue;
          int best = 0;
          for (int cta = 1; cta < ng; ++cta)
            if (load[cta] < load[best] || (load[cta] == load[best] && total[cta] < total[best])) best = cta;
          per[best].push_back(Unit{gemm | (lag << 7) | ((g + 1) << 8), tile0 + t, a0, a1 - a0});
          load[best] += a1 - a0;
          total[best] += a1 - a0;
        }
  };
  // K parts per tile: one or two entries per CTA and phase.  Every group gets the same split (the event targets count
  // units per observation), so with two streams the larger one decides.
  const int phase_groups = h->stream_split > 0 ? h->stream_split : ngroups;
  // entries per CTA and phase to aim for: one from eight observations on (measured: B = 8 11.0 against 11.8 ms per
  // launch; at B = 16 both give the same splits once O and down keep two parts), two below
  const int per_phase = h->tune.entries_per_phase > 0 ? h->tune.entries_per_phase : h->batch >= 8 ? 1 : 2;
  auto parts_for = [&](int ntiles, int stages) {
    const int want = (per_phase * ng + ntiles * phase_groups / 2) / (ntiles * phase_groups);
    return std::max(1, std::min(stages, want));
  };
  auto phase_qkv = [&](int g0, int g1) {
    std::vector<int> load(ng, 0);
    const int pq = std::min(4, parts_for(16, W / KSTAGE));
    for (int g = g0; g < g1; ++g) {
      deal(G_QKV, NKVTILES, 16, W / KSTAGE, 1, load, g, g + 1, 0);    // k / v first: attention waits for them last
      deal(G_QKV, 16, 0, W / KSTAGE, pq, load, g, g + 1, 0);
    }
  };
  auto phase = [&](int gemm, int g0, int g1, int lag) {
    std::vector<int> load(ng, 0);
    // O and down keep at least two K parts per tile: 16- and 32-stage units would leave most CTAs without work in
    // these phases (8 tiles per group)
    if (gemm == G_O) deal(G_O, W / 128, 0, QD / KSTAGE, std::max(2, parts_for(W / 128, QD / KSTAGE)), load, g0, g1, lag);
    else if (gemm == G_GU) deal(G_GU, 64, 0, W / KSTAGE, 1, load, g0, g1, lag);
    else deal(G_DOWN, W / 128, 0, FF / KSTAGE, std::max(2, parts_for(W / 128, FF / KSTAGE)), load, g0, g1, lag);
  };
  const int na = h->stream_split;
  if (na > 0) {
    // two streams of groups, A = [0, na) and B = [na, ngroups), half a layer pass apart (see row_cta in the kernel)
    phase_qkv(0, na);
    phase(G_GU, na, ngroups, 1);
    phase(G_O, 0, na, 0);
    phase(G_DOWN, na, ngroups, 1);
    phase(G_GU, 0, na, 0);
    phase_qkv(na, ngroups);
    phase(G_DOWN, 0, na, 0);
    phase(G_O, na, ngroups, 0);
  } else {
    phase_qkv(0, ngroups);
    phase(G_O, 0, ngroups, 0);
    phase(G_GU, 0, ngroups, 0);
    phase(G_DOWN, 0, ngroups, 0);
  }
  return true;
}

// Fewest GEMM CTAs any schedule works with: the 64 gate/up tiles of the one-observation schedule plus one CTA per
// row tile of the O / down projections.  plan_batch sheds groups of row CTAs until this many are left.
constexpr int MIN_GEMM_CTAS = 64 + 8;

bool build_schedule(pi05_engine* h, int ngroups = 1) {
  const int ng = h->n_gemm;
  const bool grouped = h->batch >= h->tune.grouped_from && !h->tune.latency_schedule;   // two observations still do best on the latency schedule
  // two streams of groups half a layer pass apart pay from five observations on (measured; below that they cost 1-2 %)
  h->stream_split = grouped && h->tune.two_streams && h->batch >= h->tune.streams_from && ngroups >= 2 ? (ngroups + 1) / 2 : 0;
  if (ng < MIN_GEMM_CTAS) return false;
  h->sched.assign((size_t)h->grid * MAX_UNITS, Unit{0, 0, 0, 0});
  h->sched_n.assign(h->grid, 0);
  std::vector<std::vector<Unit>> per(h->grid);
  if (!(grouped ? schedule_groups(h, per, ngroups) : schedule_one(h, per))) return false;
  for (int g = 0; g < 4; ++g) h->n_units[g] = 0;
  for (int ctaid = 0; ctaid < h->grid; ++ctaid) {
    if ((int)per[ctaid].size() > MAX_UNITS) return false;
    h->sched_n[ctaid] = (int)per[ctaid].size();
    for (size_t i = 0; i < per[ctaid].size(); ++i) {
      const Unit& un = per[ctaid][i];
      h->sched[(size_t)ctaid * MAX_UNITS + i] = un;
      if ((un.gemm >> 8) <= 1) h->n_units[un.gemm & 0x7f]++;   // units per observation: count one group's entries
    }
  }
  return true;
}

int encode_2d(pi05_engine* h, CUtensorMap* m, const void* base, uint64_t inner, uint64_t rows, uint32_t box_rows = 64) {
  EncodeTiledFn enc = get_encode();
  if (!enc) { h->last_error = "cuTensorMapEncodeTiled is not available from this driver"; return PI05_ERR_CUDA; }
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {inner * 2};
  cuuint32_t box[2] = {KATOM, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    h->last_error = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r);
    return PI05_ERR_CUDA;
  }
  return PI05_OK;
}

// K / V of attention.  The 256 dims of a token are four 64-dim segments, and the segment index is an outer dimension
// of the map, so that one copy of a box {64 dims, 64 tokens, 4 segments, 1, 1} lands as four segment blocks of
// 64 rows x 128 B (128-byte swizzle each).  `rows` tokens per page are visible (the rest read as zeros), pages are
// addressed by (layer, page); strides in BF16 elements.
int encode_kv(pi05_engine* h, CUtensorMap* m, const void* base, uint64_t rows, uint64_t layers, uint64_t pages,
              uint64_t token_stride, uint64_t layer_stride, uint64_t page_stride) {
  EncodeTiledFn enc = get_encode();
  if (!enc) { h->last_error = "cuTensorMapEncodeTiled is not available from this driver"; return PI05_ERR_CUDA; }
  cuuint64_t dims[5] = {(cuuint64_t)KATOM, rows, (cuuint64_t)(HD / KATOM), layers, pages};
  cuuint64_t strides[4] = {token_stride * 2, (cuuint64_t)KATOM * 2, layer_stride * 2, page_stride * 2};
  cuuint32_t box[5] = {KATOM, 64, HD / KATOM, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    h->last_error = "cuTensorMapEncodeTiled (attention K/V) failed with code " + std::to_string((int)r);
    return PI05_ERR_CUDA;
  }
  return PI05_OK;
}

// This layer's suffix keys / values in the workspace: [batch][50][256], described as {64, 50, 4, batch}.
int encode_suffix_kv(pi05_engine* h, CUtensorMap* m, const void* base, uint64_t planes) {
  EncodeTiledFn enc = get_encode();
  if (!enc) { h->last_error = "cuTensorMapEncodeTiled is not available from this driver"; return PI05_ERR_CUDA; }
  cuuint64_t dims[4] = {(cuuint64_t)KATOM, (cuuint64_t)T, (cuuint64_t)(HD / KATOM), planes};
  cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)KATOM * 2, (cuuint64_t)T * HD * 2};
  cuuint32_t box[4] = {KATOM, 64, HD / KATOM, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    h->last_error = "cuTensorMapEncodeTiled (suffix K/V) failed with code " + std::to_string((int)r);
    return PI05_ERR_CUDA;
  }
  return PI05_OK;
}

void default_tuning(pi05_tuning* t) {
  memset(t, 0, sizeof *t);
  t->poll_ns = 20;
  t->two_streams = 1;
  t->grouped_from = 3;
  t->streams_from = 5;
  t->clusters = 1;
}

// Clamp a caller's settings to what the engine implements.
pi05_tuning checked_tuning(const pi05_tuning& in) {
  pi05_tuning t = in;
  t.poll_ns = std::max(0, std::min(t.poll_ns, 10000));
  if (t.obs_per_mma != 1 && t.obs_per_mma != 2) t.obs_per_mma = 0;
  t.entries_per_phase = std::max(0, std::min(t.entries_per_phase, 8));
  t.grouped_from = std::max(2, t.grouped_from);
  t.streams_from = std::max(2, t.streams_from);
  t.key_groups = std::max(0, std::min(t.key_groups, (int)MAX_KEY_GROUPS));
  t.row_groups = std::max(0, std::min(t.row_groups, 3));
  return t;
}

// Everything the engine decides when it learns the batch and the prefix length: groups of row CTAs (or of keys),
// GEMM CTAs, observations per MMA, and the schedule.  Pure host arithmetic.
bool plan_batch(pi05_engine* h, int batch, int prefix_len) {
  h->batch = batch;
  // More observations keep more row CTAs busy: one group of 25 per observation in flight, as long as the GEMM
  // side keeps its 64 gate/up CTAs plus the 4 k / v CTAs.
  // One observation with a long prefix uses the extra groups differently: they split the keys of each attention.
  const int chunks = (prefix_len + 63) / 64 + 1;
  // (measured with the two-stream schedule: three groups beat two by 5-11 % at B = 5..7 and lose 4 % at B = 4)
  int groups = batch >= 5 ? 3 : batch >= 2 ? 2 : (chunks >= 8 ? 3 : chunks >= 6 ? 2 : 1);
  if (batch == 1 && h->tune.key_groups > 0) groups = h->tune.key_groups;
  if (batch > 1 && h->tune.row_groups > 0) groups = h->tune.row_groups;
  while (groups > 1 && h->grid - groups * NROW_CTAS < MIN_GEMM_CTAS) --groups;
  h->row_groups = batch > 1 ? groups : 1;
  h->key_groups = batch > 1 ? 1 : groups;
  h->n_gemm = h->grid - groups * NROW_CTAS;
  h->gn = batch == 1 ? 1 : h->tune.obs_per_mma ? h->tune.obs_per_mma : batch >= PI05_PAIRS_FROM ? 2 : 1;
  return build_schedule(h, (batch + h->gn - 1) / h->gn);
}

// The engine's description for the caller's records: geometry of the launch and the schedule of the bound batch.
void describe(pi05_engine* h) {
  char buf[1280];
  const bool grouped = h->batch >= h->tune.grouped_from && !h->tune.latency_schedule;
  snprintf(buf, sizeof buf,
           "{\"kernel\": \"pi05_chunk_kernel\", \"arch\": \"sm_100a\", \"launches_per_chunk\": 1, \"grid\": %d, "
           "\"threads\": %d, \"smem_bytes\": %d, \"gemm_ctas\": %d, \"row_ctas\": %d, \"stages\": %d, "
           "\"stage_bytes\": %d, \"units\": {\"qkv\": %d, \"o\": %d, \"gate_up\": %d, \"down\": %d}, "
           "\"mma\": \"tcgen05 cta_group::1 M128 N%d K16 bf16\", \"sync\": \"device-scope counters, bounded waits\", "
           "\"clusters_of_2\": %s, \"observations_per_mma\": %d, \"tp_rank\": %d, \"tp_size\": %d, \"schedule\": \"%s\"}",
           h->grid, THREADS, SMEM_BYTES, h->n_gemm, h->grid - h->n_gemm, h->gn == 1 ? NSTG : 3,
           W_STAGE_BYTES + h->gn * A_STAGE_BYTES, h->n_units[0], h->n_units[1], h->n_units[2], h->n_units[3], 64 * h->gn,
           h->clustered ? "true" : "false", h->gn, h->tp_rank, h->tp_size,
           !grouped ? "one observation (units serve every observation in turn)"
                    : h->stream_split > 0 ? "throughput, two streams of groups half a layer pass apart"
                                          : "throughput, one stream");
  h->config = buf;
}

bool valid_handle(pi05_handle_t h) { return h != nullptr; }

}  // namespace

// =========================================================================================== C ABI
extern "C" {

const char* pi05_error_string(int code) {
  switch (code) {
    case PI05_OK: return "ok";
    case PI05_ERR_ARGUMENT: return "invalid argument";
    case PI05_ERR_UNSUPPORTED: return "unsupported configuration";
    case PI05_ERR_CUDA: return "CUDA call failed";
    case PI05_ERR_NOT_BOUND: return "engine has no bound inputs";
    case PI05_ERR_DEVICE_TIMEOUT: return "a device-side wait timed out";
    case PI05_ERR_NO_DEVICE: return "no usable sm_100 device";
    default: return "unknown error";
  }
}

const char* pi05_last_error(pi05_handle_t h) { return valid_handle(h) ? h->last_error.c_str() : "bad handle"; }

int pi05_create(int device, int max_prefix, int max_batch, int tp_rank, int tp_size, pi05_handle_t* out) {
  if (!out) return PI05_ERR_ARGUMENT;
  *out = nullptr;
  if (device < 0 || max_prefix < 1 || max_prefix > 4096 || max_batch < 1 || tp_size < 1 || tp_rank < 0 ||
      tp_rank >= tp_size)
    return PI05_ERR_ARGUMENT;
  if (max_batch > MAXB) return PI05_ERR_UNSUPPORTED;
  if (tp_size != 1 && !((tp_size == 2 || tp_size == 4 || tp_size == 8) && max_batch == 1)) return PI05_ERR_UNSUPPORTED;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { cudaGetLastError(); return PI05_ERR_NO_DEVICE; }
  if (device >= ndev) return PI05_ERR_ARGUMENT;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); return PI05_ERR_NO_DEVICE; }
  if (prop.major != 10) return PI05_ERR_NO_DEVICE;
  pi05_engine* h = new (std::nothrow) pi05_engine();
  if (!h) return PI05_ERR_ARGUMENT;
  h->device = device;
  h->sms = prop.multiProcessorCount;
  h->grid = h->sms;
  h->row_groups = 1;
  h->n_gemm = h->grid - NROW_CTAS;
  h->max_prefix = max_prefix;
  h->max_batch = max_batch;
  h->tp_rank = tp_rank;
  h->tp_size = tp_size;
  default_tuning(&h->tune);
  if (!build_schedule(h)) { delete h; return PI05_ERR_UNSUPPORTED; }
  build_layout(h);
  DeviceGuard guard(device);
  if (!guard.ok) { delete h; return PI05_ERR_CUDA; }
  cudaError_t e = cudaSuccess;
  for (const void* kern : kAllKernels) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) { cudaGetLastError(); delete h; return PI05_ERR_CUDA; }
  }
  int coop = 0, blocks = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, k_traced::pi05_chunk_kernel, THREADS, SMEM_BYTES);
  if (e != cudaSuccess || blocks < 1 || !coop) { cudaGetLastError(); delete h; return PI05_ERR_UNSUPPORTED; }
  {
    // Clusters of two CTAs when the whole grid fits that way: the kernel uses no cluster feature, but the launch then
    // places consecutive blocks on the two SMs of a TPC, which measured ~1 % faster than the plain cooperative
    // launch's placement.  The tuning setting `clusters = 0` selects the plain launch.
    bool want = h->grid % 2 == 0;
    for (const void* kern : kAllKernels) {
      if (!want) break;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof cfg);
      cfg.gridDim = dim3(h->grid); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM_BYTES;
      cfg.attrs = &attr; cfg.numAttrs = 1;
      int nclusters = 0;
      if (cudaOccupancyMaxActiveClusters(&nclusters, kern, &cfg) != cudaSuccess || nclusters < h->grid / 2) {
        cudaGetLastError();
        want = false;
      }
    }
    h->can_cluster = want;
    h->clustered = want;
  }
  // marks the end of this handle's last launch: pi05_status and a re-bind wait for it instead of for the whole device
  e = cudaEventCreateWithFlags(&h->done, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->side, cudaStreamNonBlocking);
  if (e != cudaSuccess) { cudaGetLastError(); if (h->done) cudaEventDestroy(h->done); delete h; return PI05_ERR_CUDA; }
  describe(h);
  *out = h;
  return PI05_OK;
}

int pi05_tuning_defaults(pi05_tuning* t) {
  if (!t) return PI05_ERR_ARGUMENT;
  default_tuning(t);
  return PI05_OK;
}

int pi05_tune(pi05_handle_t h, const pi05_tuning* t) {
  if (!valid_handle(h) || !t) return PI05_ERR_ARGUMENT;
  h->tune = checked_tuning(*t);
  h->clustered = h->can_cluster && h->tune.clusters != 0;
  h->bound = false;              // the schedule and the launch shape are chosen at bind
  describe(h);
  return PI05_OK;
}

int pi05_workspace_bytes(pi05_handle_t h, size_t* bytes) {
  if (!valid_handle(h) || !bytes) return PI05_ERR_ARGUMENT;
  *bytes = h->ws_bytes;
  return PI05_OK;
}

int pi05_bind(pi05_handle_t h, const void* const inputs[PI05_NUM_INPUTS], int prefix_len, int batch, void* actions,
              void* workspace, size_t workspace_bytes) {
  if (!valid_handle(h) || !inputs) return PI05_ERR_ARGUMENT;
  if (batch < 1 || batch > MAXB || prefix_len < 1) return PI05_ERR_ARGUMENT;
  if (!inputs[22] || !inputs[23]) { h->last_error = "null input pointer"; return PI05_ERR_ARGUMENT; }
  // dense [batch][18][P][1][256]: one page per observation
  int table[MAXB];
  for (int b = 0; b < batch; ++b) table[b] = b;
  pi05_kv_view kv;
  kv.k = inputs[22]; kv.v = inputs[23];
  kv.token_stride = HD; kv.layer_stride = (long long)prefix_len * HD; kv.page_stride = (long long)NL * prefix_len * HD;
  kv.page_tokens = prefix_len; kv.num_pages = batch; kv.pages_per_obs = 1; kv.page_table = table;
  return pi05_bind_view(h, inputs, &kv, prefix_len, batch, actions, workspace, workspace_bytes);
}

int pi05_bind_view(pi05_handle_t h, const void* const inputs[PI05_NUM_INPUTS], const pi05_kv_view* kv, int prefix_len,
                   int batch, void* actions, void* workspace, size_t workspace_bytes) {
  if (!valid_handle(h) || !inputs || !kv || !actions || !workspace) return PI05_ERR_ARGUMENT;
  if (batch < 1) return PI05_ERR_ARGUMENT;
  if (batch > h->max_batch) return PI05_ERR_UNSUPPORTED;
  if (prefix_len < 1 || prefix_len > h->max_prefix) return PI05_ERR_ARGUMENT;
  if (workspace_bytes < h->ws_bytes) { h->last_error = "workspace too small"; return PI05_ERR_ARGUMENT; }
  {
    // the view of the prefix cache
    const int max_pages = (h->max_prefix + 63) / 64;
    if (!kv->k || !kv->v || !kv->page_table) { h->last_error = "null pointer in the prefix cache view"; return PI05_ERR_ARGUMENT; }
    if ((reinterpret_cast<uintptr_t>(kv->k) & 15) || (reinterpret_cast<uintptr_t>(kv->v) & 15)) {
      h->last_error = "prefix cache pools must be 16-byte aligned";
      return PI05_ERR_ARGUMENT;
    }
    if (kv->token_stride < HD || kv->layer_stride < 0 || kv->page_stride < 0 || (kv->token_stride & 7) ||
        (kv->layer_stride & 7) || (kv->page_stride & 7)) {
      h->last_error = "prefix cache strides must be multiples of 8 elements (token stride >= 256)";
      return PI05_ERR_ARGUMENT;
    }
    if (kv->page_tokens < 1 || kv->num_pages < 1 || kv->pages_per_obs < 1 || kv->pages_per_obs > max_pages ||
        (kv->pages_per_obs > 1 && kv->page_tokens % 64 != 0) ||
        (long long)kv->pages_per_obs * kv->page_tokens < prefix_len) {
      h->last_error = "prefix cache pages do not cover the prefix (page_tokens must be a multiple of 64 with several pages)";
      return PI05_ERR_ARGUMENT;
    }
    if ((long long)batch * kv->pages_per_obs > MAX_PAGE_ENTRIES) {
      h->last_error = "page table too large (batch x pages per observation > 1024)";
      return PI05_ERR_UNSUPPORTED;
    }
    for (int i = 0; i < batch * kv->pages_per_obs; ++i)
      if (kv->page_table[i] < 0 || kv->page_table[i] >= kv->num_pages) {
        h->last_error = "page table entry " + std::to_string(i) + " is outside the pool";
        return PI05_ERR_ARGUMENT;
      }
  }
  for (int i = 0; i < PI05_NUM_INPUTS; ++i) {
    if (i == 22 || i == 23) continue;   // superseded by the view
    if (!inputs[i]) { h->last_error = "null input pointer"; return PI05_ERR_ARGUMENT; }
    if (i != 24 && (reinterpret_cast<uintptr_t>(inputs[i]) & 15)) {
      h->last_error = "input " + std::to_string(i) + " is not 16-byte aligned";
      return PI05_ERR_ARGUMENT;
    }
  }
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(actions) & 15)) {
    h->last_error = "workspace must be 256-byte and actions 16-byte aligned";
    return PI05_ERR_ARGUMENT;
  }
  DeviceGuard guard(h->device);
  if (!guard.ok) return PI05_ERR_CUDA;
  h->bound = false;
  if (h->in_flight) {
    // a launch of this handle may still be running out of the workspace that is about to be cleared and re-described
    cudaError_t e = cudaEventSynchronize(h->done);
    if (e != cudaSuccess) return fail_cuda(h, "cudaEventSynchronize", e);
  }
  for (int i = 0; i < PI05_NUM_INPUTS; ++i) h->inputs[i] = inputs[i];
  h->inputs[22] = kv->k; h->inputs[23] = kv->v;
  h->pages_per_obs = kv->pages_per_obs;
  h->page_tokens = kv->page_tokens;
  h->actions = actions;
  h->ws = static_cast<uint8_t*>(workspace);
  h->prefix = prefix_len;
  h->batch = batch;
  h->tp_base = 0;                 // the workspace, counters included, is cleared below
  if (!plan_batch(h, batch, prefix_len)) { h->last_error = "no schedule for this GPU"; return PI05_ERR_UNSUPPORTED; }
  describe(h);
  cudaError_t e = cudaMemset(workspace, 0, h->ws_bytes);
  if (e != cudaSuccess) return fail_cuda(h, "cudaMemset(workspace)", e);
  e = cudaMemcpy(region_ptr<void>(h, "sched"), h->sched.data(), h->sched.size() * sizeof(Unit), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return fail_cuda(h, "cudaMemcpy(schedule)", e);
  e = cudaMemcpy(region_ptr<void>(h, "sched_n"), h->sched_n.data(), h->sched_n.size() * sizeof(int), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return fail_cuda(h, "cudaMemcpy(schedule)", e);
  int rc;
  if ((rc = encode_2d(h, &h->maps.wq, inputs[8], W, (uint64_t)NL * QD))) return rc;
  if ((rc = encode_2d(h, &h->maps.wk, inputs[9], W, (uint64_t)NL * HD))) return rc;
  if ((rc = encode_2d(h, &h->maps.wv, inputs[10], W, (uint64_t)NL * HD))) return rc;
  if ((rc = encode_2d(h, &h->maps.wo, inputs[11], QD, (uint64_t)NL * W))) return rc;
  if ((rc = encode_2d(h, &h->maps.wg, inputs[12], W, (uint64_t)NL * FF))) return rc;
  if ((rc = encode_2d(h, &h->maps.wu, inputs[13], W, (uint64_t)NL * FF))) return rc;
  if ((rc = encode_2d(h, &h->maps.wd, inputs[14], FF, (uint64_t)NL * W))) return rc;
  if ((rc = encode_2d(h, &h->maps.an_attn, region_ptr<void>(h, "an_attn"), W, (uint64_t)T * batch * AN_COPIES, A_BOX_ROWS))) return rc;
  if ((rc = encode_2d(h, &h->maps.an_ffn, region_ptr<void>(h, "an_ffn"), W, (uint64_t)T * batch * AN_COPIES, A_BOX_ROWS))) return rc;
  if ((rc = encode_2d(h, &h->maps.attn, region_ptr<void>(h, "attn"), QD, (uint64_t)T * batch, A_BOX_ROWS))) return rc;
  if ((rc = encode_2d(h, &h->maps.act, region_ptr<void>(h, "act"), FF, (uint64_t)T * batch, A_BOX_ROWS))) return rc;
  if ((rc = encode_suffix_kv(h, &h->maps.sk, region_ptr<void>(h, "k"), (uint64_t)batch))) return rc;
  if ((rc = encode_suffix_kv(h, &h->maps.sv, region_ptr<void>(h, "v"), (uint64_t)batch))) return rc;
  {
    // full pages, and the last page of an observation cut at its last valid token
    const uint64_t full_rows = (uint64_t)kv->page_tokens;
    const uint64_t tail_rows = (uint64_t)(prefix_len - (prefix_len - 1) / kv->page_tokens * kv->page_tokens);
    const void* pools[2] = {kv->k, kv->v};
    CUtensorMap* full[2] = {&h->maps.pk, &h->maps.pv};
    CUtensorMap* tail[2] = {&h->maps.pk_tail, &h->maps.pv_tail};
    for (int i = 0; i < 2; ++i) {
      if ((rc = encode_kv(h, full[i], pools[i], full_rows, NL, (uint64_t)kv->num_pages, (uint64_t)kv->token_stride,
                          (uint64_t)kv->layer_stride, (uint64_t)kv->page_stride))) return rc;
      if ((rc = encode_kv(h, tail[i], pools[i], tail_rows, NL, (uint64_t)kv->num_pages, (uint64_t)kv->token_stride,
                          (uint64_t)kv->layer_stride, (uint64_t)kv->page_stride))) return rc;
    }
  }
  e = cudaMemcpy(region_ptr<void>(h, "page_table"), kv->page_table, (size_t)batch * kv->pages_per_obs * sizeof(int),
                 cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return fail_cuda(h, "cudaMemcpy(page table)", e);
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(h, "cudaDeviceSynchronize", e);
  h->bound = true;
  return PI05_OK;
}

int pi05_refresh(pi05_handle_t h) {
  if (!valid_handle(h)) return PI05_ERR_ARGUMENT;
  return h->bound ? PI05_OK : PI05_ERR_NOT_BOUND;
}

int pi05_debug(pi05_handle_t h, int max_stage, long long wait_limit_cycles, int drop_event) {
  if (!valid_handle(h) || drop_event >= NEVENTS) return PI05_ERR_ARGUMENT;
  h->drop_event = drop_event < 0 ? -1 : drop_event;
  h->max_stage = max_stage < 0 ? 0x7fffffff : max_stage;
  if (wait_limit_cycles > 0) h->wait_limit = wait_limit_cycles;
  return PI05_OK;
}

int pi05_launch(pi05_handle_t h, int n_steps, int n_layers, void* stream, unsigned long long* stamps) {
  if (!valid_handle(h)) return PI05_ERR_ARGUMENT;
  if (!h->bound) return PI05_ERR_NOT_BOUND;
  if (n_steps < 1 || n_steps > NS || n_layers < 1 || n_layers > NL) return PI05_ERR_ARGUMENT;
  DeviceGuard guard(h->device);
  if (!guard.ok) return PI05_ERR_CUDA;
  Params p;
  memset(&p, 0, sizeof p);
  p.maps = h->maps;
  const void* const* in = h->inputs;
  p.ain_w = (const float*)in[0]; p.ain_b = (const float*)in[1];
  p.tin_w = (const float*)in[2]; p.tin_b = (const float*)in[3];
  p.tout_w = (const float*)in[4]; p.tout_b = (const float*)in[5];
  p.aout_w = (const float*)in[6]; p.aout_b = (const float*)in[7];
  p.attn_nw = (const float*)in[15]; p.attn_nb = (const float*)in[16];
  p.ffn_nw = (const float*)in[17]; p.ffn_nb = (const float*)in[18];
  p.fin_nw = (const float*)in[19]; p.fin_nb = (const float*)in[20];
  p.wq = (const __nv_bfloat16*)in[8]; p.wk = (const __nv_bfloat16*)in[9]; p.wv = (const __nv_bfloat16*)in[10];
  p.wo = (const __nv_bfloat16*)in[11]; p.wg = (const __nv_bfloat16*)in[12]; p.wu = (const __nv_bfloat16*)in[13];
  p.wd = (const __nv_bfloat16*)in[14];
  ObsPtrs& o = p.ob;
  o.noise = (const float*)in[21];

  o.prefix_mask = (const uint8_t*)in[24];
  o.actions = (float*)h->actions;
  o.x = region_ptr<float>(h, "x"); o.o_acc = region_ptr<float>(h, "o_acc"); o.d_acc = region_ptr<float>(h, "d_acc");
  o.qkv_acc = region_ptr<float>(h, "qkv_acc");
  o.rope = region_ptr<uint32_t>(h, "rope"); o.rope2 = region_ptr<uint32_t>(h, "rope2");
  o.h = region_ptr<__nv_bfloat16>(h, "h"); o.an_attn = region_ptr<__nv_bfloat16>(h, "an_attn");
  o.an_ffn = region_ptr<__nv_bfloat16>(h, "an_ffn");
  o.k = region_ptr<__nv_bfloat16>(h, "k"); o.v = region_ptr<__nv_bfloat16>(h, "v");
  o.attn = region_ptr<__nv_bfloat16>(h, "attn"); o.act = region_ptr<__nv_bfloat16>(h, "act");
  o.b = 0;
  p.ctrl = region_ptr<unsigned int>(h, "ctrl");
  p.temb = region_ptr<float>(h, "temb"); p.hid = region_ptr<float>(h, "hid"); p.cond = region_ptr<float>(h, "cond");
  p.mod = region_ptr<float>(h, "mod");
  p.sched = region_ptr<Unit>(h, "sched"); p.sched_n = region_ptr<int>(h, "sched_n");
  p.stamps = stamps;
  p.wait_limit = h->wait_limit;
  p.batch = h->batch;
  p.prefix = h->prefix; p.n_steps = n_steps; p.n_layers = n_layers; p.max_stage = h->max_stage;
  p.n_gemm_ctas = h->n_gemm;
  p.row_groups = h->row_groups;
  p.key_groups = h->key_groups;
  p.att_part = region_ptr<float>(h, "att_part");
  p.page_table = region_ptr<int>(h, "page_table");
  p.pages_per_obs = h->pages_per_obs; p.page_tokens = h->page_tokens;
  p.tp_rank = h->tp_rank; p.tp_size = h->tp_size; p.tp_base = h->tp_base;
  if (h->tp_size > 1) {
    p.tp_recv = region_ptr<float>(h, "tp_recv");
    p.tp_flags = region_ptr<unsigned int>(h, "tp_flags");
    for (int r = 0; r < h->tp_size; ++r) {
      if (r == h->tp_rank) continue;
      if (!h->tp_peer_recv[r]) { h->last_error = "tensor parallel: peer " + std::to_string(r) + " is not attached"; return PI05_ERR_NOT_BOUND; }
      p.tp_peer_recv[r] = h->tp_peer_recv[r];
      p.tp_peer_flags[r] = h->tp_peer_flags[r];
    }
  }
  p.drop_event = h->drop_event;
  p.poll_ns = h->tune.poll_ns;
  for (int g = 0; g < 4; ++g) p.n_units[g] = h->n_units[g];
  p.cta_perm = h->tune.cta_perm && h->grid % 2 == 0 ? 1 : 0;
  // the throughput schedule runs the O units of every group before any gate/up unit, so the row CTAs do all their
  // attentions first; the latency schedule interleaves the residual of one observation with the attention of the next
  p.row_order = h->batch >= h->tune.grouped_from && !h->tune.latency_schedule ? 1 : 0;
  p.stream_split = h->stream_split;
  const double dt = -1.0 / NS;
  for (int s = 0; s < NS; ++s) p.t_steps[s] = (float)(1.0 + s * dt);
  p.dt = (float)dt;
  void* args[] = {&p};
  // stamps or a debug control wanted: the traced build; otherwise the build without that code, specialised for
  // one observation when there is only one, and with two or four observations side by side in every MMA when
  // there are several (a weight stage in shared memory then serves all of them)
  const bool debug = stamps != nullptr || h->max_stage != 0x7fffffff || h->drop_event >= 0;
  const int gn = h->gn;
  if (debug && h->tp_size > 1) {
    h->last_error = "stamps and debug controls are not available in a tensor-parallel engine";
    return PI05_ERR_UNSUPPORTED;
  }
  if (debug && h->stream_split > 0 && (h->max_stage != 0x7fffffff)) {
    h->last_error = "the stage limit is not available with the two-stream schedule of a batch (tune the engine with two_streams = 0)";
    return PI05_ERR_UNSUPPORTED;
  }
  if (debug && gn != 1) {   // the traced build runs one observation per MMA; the bound schedule is for groups of gn
    h->last_error = "stamps and debug controls need one observation per MMA (tuning setting obs_per_mma 0 or 1)";
    return PI05_ERR_UNSUPPORTED;
  }
  const void* kern = debug ? (const void*)k_traced::pi05_chunk_kernel
                     : h->tp_size > 1 ? (const void*)k_tp::pi05_chunk_kernel
                     : h->batch == 1 ? (const void*)k_plain::pi05_chunk_kernel
                     : gn == 2 ? (const void*)k_pairs::pi05_chunk_kernel
                               : (const void*)k_batched::pi05_chunk_kernel;
  cudaError_t e;
  if (h->clustered) {
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeCooperative;
    attrs[0].val.cooperative = 1;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = 2; attrs[1].val.clusterDim.y = 1; attrs[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(h->grid); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = (cudaStream_t)stream; cfg.attrs = attrs; cfg.numAttrs = 2;
    e = cudaLaunchKernelExC(&cfg, kern, args);
  } else {
    e = cudaLaunchCooperativeKernel(kern, dim3(h->grid), dim3(THREADS), args, SMEM_BYTES, (cudaStream_t)stream);
  }
  if (e != cudaSuccess) return fail_cuda(h, "kernel launch", e);
  h->launches++;
  h->tp_base += (unsigned)((h->tp_size - 1) * n_steps * n_layers);   // two exchanges per layer pass, one counter each
  e = cudaEventRecord(h->done, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail_cuda(h, "cudaEventRecord", e);
  h->in_flight = true;
  return PI05_OK;
}

// Reads (and, when set, clears) the status word of a handle whose last launch has completed.
static int read_status(pi05_engine* h, int* code, int* where) {
  unsigned int st[2] = {0, 0};
  cudaError_t e = cudaMemcpyAsync(st, h->ws, sizeof st, cudaMemcpyDeviceToHost, h->side);
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->side);
  if (e != cudaSuccess) return fail_cuda(h, "copy of the status word", e);
  *code = (int)st[0];
  *where = (int)st[1];
  if (st[0]) {
    e = cudaMemsetAsync(h->ws, 0, CTRL_BYTES, h->side);   // status and every counter: the next launch starts clean
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->side);
    if (e != cudaSuccess) return fail_cuda(h, "clearing of the status word", e);
    return PI05_ERR_DEVICE_TIMEOUT;
  }
  return PI05_OK;
}

int pi05_status(pi05_handle_t h, int* code, int* where) {
  if (!valid_handle(h) || !code || !where) return PI05_ERR_ARGUMENT;
  if (!h->ws) return PI05_ERR_NOT_BOUND;
  DeviceGuard guard(h->device);
  if (!guard.ok) return PI05_ERR_CUDA;
  // wait for this handle's last launch only (other handles and streams of the GPU keep running)
  cudaError_t e = h->in_flight ? cudaEventSynchronize(h->done) : cudaSuccess;
  if (e != cudaSuccess) return fail_cuda(h, "cudaEventSynchronize", e);
  h->in_flight = false;
  return read_status(h, code, where);
}

int pi05_workspace_region(pi05_handle_t h, const char* name, size_t* offset, size_t* bytes) {
  if (!valid_handle(h) || !name || !offset || !bytes) return PI05_ERR_ARGUMENT;
  const Region* r = find_region(h, name);
  if (!r) return PI05_ERR_ARGUMENT;
  *offset = r->off;
  *bytes = r->bytes;
  return PI05_OK;
}

int pi05_schedule_plan(int sms, int batch, int prefix_len, const pi05_tuning* tuning, int* entries, int capacity,
                       int* count, int info[PI05_PLAN_INFO]) {
  return pi05_schedule_plan_tp(sms, batch, prefix_len, 0, 1, tuning, entries, capacity, count, info);
}

int pi05_schedule_plan_tp(int sms, int batch, int prefix_len, int tp_rank, int tp_size, const pi05_tuning* tuning,
                          int* entries, int capacity, int* count, int info[PI05_PLAN_INFO]) {
  if (sms < 1 || sms > 1024 || batch < 1 || batch > MAXB || prefix_len < 1 || capacity < 0 || (capacity > 0 && !entries) ||
      !count || !info || tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size)
    return PI05_ERR_ARGUMENT;
  if (tp_size != 1 && !((tp_size == 2 || tp_size == 4 || tp_size == 8) && batch == 1)) return PI05_ERR_UNSUPPORTED;
  pi05_engine h;                 // host-side state only: nothing here touches a device
  h.grid = sms;
  h.n_gemm = sms - NROW_CTAS;
  h.tp_rank = tp_rank; h.tp_size = tp_size;
  default_tuning(&h.tune);
  if (tuning) h.tune = checked_tuning(*tuning);
  if (h.n_gemm < 1 || !plan_batch(&h, batch, prefix_len)) return PI05_ERR_UNSUPPORTED;
  info[0] = h.n_gemm; info[1] = h.row_groups; info[2] = h.key_groups; info[3] = h.gn;
  info[4] = (batch + h.gn - 1) / h.gn; info[5] = h.stream_split;
  for (int g = 0; g < 4; ++g) info[6 + g] = h.n_units[g];
  int n = 0;
  for (int cta = 0; cta < h.grid; ++cta)
    for (int i = 0; i < h.sched_n[cta]; ++i, ++n) {
      if (n >= capacity) continue;           // keep counting: *count says how many there are
      const Unit& un = h.sched[(size_t)cta * MAX_UNITS + i];
      int* e = entries + (size_t)n * PI05_PLAN_ENTRY;
      e[0] = cta; e[1] = un.gemm & 0x7f; e[2] = (un.gemm >> 7) & 1; e[3] = (un.gemm >> 8) - 1;
      e[4] = un.tile; e[5] = un.k0; e[6] = un.nk;
    }
  *count = n;
  return PI05_OK;
}

// ---- tensor parallel: how the ranks learn where each other's receive buffers are
namespace {
struct TpHandle {                 // what pi05_tp_export writes: PI05_TP_HANDLE_BYTES
  cudaIpcMemHandle_t ipc;         // the allocation that holds the workspace
  unsigned long long offset;      // of the workspace inside that allocation
  unsigned long long ws_bytes;
};
static_assert(sizeof(TpHandle) <= PI05_TP_HANDLE_BYTES, "handle size");

int tp_attach_at(pi05_engine* h, int peer, uint8_t* peer_ws) {
  const Region* recv = find_region(h, "tp_recv");
  const Region* flags = find_region(h, "tp_flags");
  if (!recv || !flags) return PI05_ERR_UNSUPPORTED;
  h->tp_peer_recv[peer] = reinterpret_cast<float*>(peer_ws + recv->off);
  h->tp_peer_flags[peer] = reinterpret_cast<unsigned int*>(peer_ws + flags->off);
  return PI05_OK;
}
}  // namespace

int pi05_tp_export(pi05_handle_t h, void* out, size_t out_bytes) {
  if (!valid_handle(h) || !out || out_bytes < PI05_TP_HANDLE_BYTES) return PI05_ERR_ARGUMENT;
  if (h->tp_size < 2) return PI05_ERR_UNSUPPORTED;
  if (!h->bound) return PI05_ERR_NOT_BOUND;
  DeviceGuard guard(h->device);
  if (!guard.ok) return PI05_ERR_CUDA;
  TpHandle th;
  memset(&th, 0, sizeof th);
  // the workspace may sit anywhere inside a larger allocation of the caller's allocator: export that allocation and
  // the offset
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || !fn) {
    h->last_error = "cuMemGetAddressRange is not available from this driver";
    return PI05_ERR_CUDA;
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(h->ws)) != CUDA_SUCCESS) {
    h->last_error = "cuMemGetAddressRange failed on the workspace";
    return PI05_ERR_CUDA;
  }
  cudaError_t e = cudaIpcGetMemHandle(&th.ipc, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) return fail_cuda(h, "cudaIpcGetMemHandle(workspace)", e);
  th.offset = reinterpret_cast<CUdeviceptr>(h->ws) - base;
  th.ws_bytes = h->ws_bytes;
  memset(out, 0, PI05_TP_HANDLE_BYTES);
  memcpy(out, &th, sizeof th);
  return PI05_OK;
}

int pi05_tp_attach(pi05_handle_t h, int peer_rank, const void* exported) {
  if (!valid_handle(h) || !exported) return PI05_ERR_ARGUMENT;
  if (h->tp_size < 2) return PI05_ERR_UNSUPPORTED;
  if (peer_rank < 0 || peer_rank >= h->tp_size || peer_rank == h->tp_rank) return PI05_ERR_ARGUMENT;
  TpHandle th;
  memcpy(&th, exported, sizeof th);
  if (th.ws_bytes != h->ws_bytes) { h->last_error = "the peer's workspace has another layout"; return PI05_ERR_ARGUMENT; }
  DeviceGuard guard(h->device);
  if (!guard.ok) return PI05_ERR_CUDA;
  if (h->tp_opened[peer_rank]) { cudaIpcCloseMemHandle(h->tp_opened[peer_rank]); h->tp_opened[peer_rank] = nullptr; }
  void* base = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&base, th.ipc, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail_cuda(h, "cudaIpcOpenMemHandle(peer workspace)", e);
  h->tp_opened[peer_rank] = base;
  return tp_attach_at(h, peer_rank, static_cast<uint8_t*>(base) + th.offset);
}

int pi05_tp_attach_pointer(pi05_handle_t h, int peer_rank, void* peer_workspace) {
  if (!valid_handle(h) || !peer_workspace) return PI05_ERR_ARGUMENT;
  if (h->tp_size < 2) return PI05_ERR_UNSUPPORTED;
  if (peer_rank < 0 || peer_rank >= h->tp_size || peer_rank == h->tp_rank) return PI05_ERR_ARGUMENT;
  return tp_attach_at(h, peer_rank, static_cast<uint8_t*>(peer_workspace));
}

const char* pi05_config_json(pi05_handle_t h) { return valid_handle(h) ? h->config.c_str() : "{}"; }

int pi05_launch_count(pi05_handle_t h, unsigned long long* count) {
  if (!valid_handle(h) || !count) return PI05_ERR_ARGUMENT;
  *count = h->launches;
  return PI05_OK;
}

int pi05_destroy(pi05_handle_t h) {
  if (!valid_handle(h)) return PI05_ERR_ARGUMENT;
  if (h->done) {
    DeviceGuard guard(h->device);
    cudaEventDestroy(h->done);
    if (h->side) cudaStreamDestroy(h->side);
    for (int r = 0; r < MAX_TP; ++r)
      if (h->tp_opened[r]) cudaIpcCloseMemHandle(h->tp_opened[r]);
  }
  delete h;
  return PI05_OK;
}

}  // extern "C"

// =========================================================================================== no-allocation entry
// Scratch for pi05_chunk_static(): the whole workspace of one engine lives in this file-scope device array
// instead of a caller-allocated buffer.  Every GPU that loads the library holds these bytes until the process
// exits.  Host code must not hand this name to a kernel: on the host it is only a stand-in for the symbol; the
// device address comes from cudaGetSymbolAddress() below.
static __device__ __align__(256) unsigned char g_pi05_static_scratch[PI05_STATIC_SCRATCH_BYTES];

namespace {

struct StaticSlot {
  pi05_handle_t h = nullptr;        // host-side engine state of this device (created on the first call)
  void* scratch = nullptr;          // device address of g_pi05_static_scratch on this device
  const void* inputs[PI05_NUM_INPUTS] = {};
  void* actions = nullptr;
  int prefix = 0;
  bool bound = false;
};
constexpr int MAX_STATIC_DEVICES = 64;
StaticSlot g_static_slots[MAX_STATIC_DEVICES];
std::mutex g_static_mutex;

}  // namespace

extern "C" int pi05_chunk_static(int device, const void* const inputs[PI05_NUM_INPUTS], int prefix_len, void* actions,
                                 int n_steps, int n_layers, void* stream) {
  if (device < 0 || device >= MAX_STATIC_DEVICES || !inputs || !actions) return PI05_ERR_ARGUMENT;
  if (prefix_len < 1) return PI05_ERR_ARGUMENT;
  if (prefix_len > PI05_STATIC_MAX_PREFIX) return PI05_ERR_UNSUPPORTED;   // beyond the stated maximum
  if (n_steps < 1 || n_steps > NS || n_layers < 1 || n_layers > NL) return PI05_ERR_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticSlot& slot = g_static_slots[device];
  if (!slot.h) {
    // Set-up, once per device: host-side engine state, then the device address of the static array, taken with
    // that device current.  No device memory is allocated anywhere on this path.
    pi05_handle_t h = nullptr;
    int rc = pi05_create(device, PI05_STATIC_MAX_PREFIX, 1, 0, 1, &h);
    if (rc != PI05_OK) return rc;
    size_t need = 0;
    pi05_workspace_bytes(h, &need);
    if (need > (size_t)PI05_STATIC_SCRATCH_BYTES) {   // e.g. a part with many more SMs: the schedule would not fit
      pi05_destroy(h);
      return PI05_ERR_UNSUPPORTED;
    }
    void* ptr = nullptr;
    {
      DeviceGuard guard(device);
      if (!guard.ok) { pi05_destroy(h); return PI05_ERR_CUDA; }
      cudaError_t e = cudaGetSymbolAddress(&ptr, g_pi05_static_scratch);
      if (e != cudaSuccess || ptr == nullptr) { cudaGetLastError(); pi05_destroy(h); return PI05_ERR_CUDA; }
    }
    slot.h = h;
    slot.scratch = ptr;
    slot.bound = false;
  }
  if (slot.h->in_flight) {
    // An earlier call whose kernel has finished by now: look at the status word it left before this call clears it.
    // (A kernel whose bounded wait gave up fills its actions with NaN and leaves a code here; this is where the caller
    // of this entry point learns of it.  A call that is still running is not waited for.)
    DeviceGuard guard(device);
    if (!guard.ok) return PI05_ERR_CUDA;
    if (cudaEventQuery(slot.h->done) == cudaSuccess) {
      slot.h->in_flight = false;
      int code = 0, where = 0;
      const int rc = read_status(slot.h, &code, &where);
      if (rc != PI05_OK) return rc;
    } else {
      cudaGetLastError();
    }
  }
  bool same = slot.bound && slot.prefix == prefix_len && slot.actions == actions;
  for (int i = 0; same && i < PI05_NUM_INPUTS; ++i) same = slot.inputs[i] == inputs[i];
  if (!same) {
    // New tensors or a new prefix length: re-encode the TMA descriptors and clear the scratch.  The bind first waits
    // for the last launch out of this array (whatever stream it is on) and synchronises the device at its end.
    slot.bound = false;
    int rc = pi05_bind(slot.h, inputs, prefix_len, 1, actions, slot.scratch, (size_t)PI05_STATIC_SCRATCH_BYTES);
    if (rc != PI05_OK) return rc;
    for (int i = 0; i < PI05_NUM_INPUTS; ++i) slot.inputs[i] = inputs[i];
    slot.actions = actions;
    slot.prefix = prefix_len;
    slot.bound = true;
  }
  {
    // The array keeps whatever the last call left.  What has to start at zero is the control block (status word
    // and stage counters; an aborted call could leave them dirty); the kernel clears its accumulators itself.
    DeviceGuard guard(device);
    if (!guard.ok) return PI05_ERR_CUDA;
    cudaError_t e = cudaMemsetAsync(slot.scratch, 0, CTRL_BYTES, (cudaStream_t)stream);
    if (e != cudaSuccess) { cudaGetLastError(); return PI05_ERR_CUDA; }
  }
  return pi05_launch(slot.h, n_steps, n_layers, stream, nullptr);
}

