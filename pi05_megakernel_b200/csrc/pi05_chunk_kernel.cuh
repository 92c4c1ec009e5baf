// The chunk kernel and all of its device code.  This file has no include guard on purpose: the translation unit
// includes it once per variant, inside a namespace of its own, with two macros set:
//   PI05_TRACE    1: the kernel writes globaltimer stamps when given a stamp buffer and honours the debug controls
//                    (stage limit, withheld signal); 0: none of that code exists (the single-thread issue loops
//                    are sensitive to every instruction: the production kernel is ~3 % faster without it)
//   PI05_BATCHED  1: any number of observations per launch; 0: exactly one, and all per-observation pointer
//                    arithmetic and loops fold away
//   PI05_TP       1: tensor parallel, one observation shared by several GPUs: every rank runs the query heads and
//                    MLP columns its schedule names, and the partial sums of the O and down projections are exchanged
//                    between the ranks' row CTAs over NVLink (peer stores and system-scope counters) inside the
//                    gated-residual operation; 0: none of that code exists
//   PI05_GN       observations per MMA (1 or 2): the GEMM CTAs put the activations of GN observations side by
//                    side on the N side of one MMA (N = 64 * GN), so a weight stage in shared memory is fetched
//                    once for all of them.  The activation half of a stage grows to GN x 16 KB and the ring keeps
//                    192 KB: 4 or 3 stages.  Row CTAs and counters stay per observation.  (Four observations per
//                    MMA leave a ring of two stages and measured slower than two at every batch size.)
#if PI05_TRACE
#define PI05_MAXSTAGE(p) ((p).max_stage)
#define PI05_DROP(p) ((p).drop_event)
#else
#define PI05_MAXSTAGE(p) 0x7fffffff
#define PI05_DROP(p) (-1)
#endif
#if PI05_BATCHED
#define PI05_NB(p) ((p).batch)
#define PI05_NG(p) ((p).row_groups)
#else
#define PI05_NB(p) 1
#define PI05_NG(p) 1
#endif

constexpr int GN = PI05_GN;
static_assert(GN == 1 || GN == 2, "observations per MMA");
static_assert(GN == 1 || PI05_BATCHED, "several observations per MMA only in a batched build");
constexpr int V_A_ATOM = GN * A_ATOM_BYTES;            // 64 * GN token rows x 64 k: observation g's box at g * A_ATOM_BYTES
constexpr int V_STAGE_ALL = W_STAGE_BYTES + 2 * V_A_ATOM;
constexpr int V_NSTG = GN == 1 ? 4 : 3;
constexpr int V_TMEM_COLS = 2 * 64 * GN;               // two accumulators of 64 * GN columns
static_assert(V_NSTG * V_STAGE_ALL <= OFF_STAGE && V_NSTG <= NSTG && V_TMEM_COLS <= 512, "ring / TMEM capacity");
#define PI05_NGRP(p) ((PI05_NB(p) + GN - 1) / GN)      // groups of observations that share MMAs

__device__ __constant__ int kGemmStage[4] = {ST_QKV, ST_O, ST_GU, ST_DOWN};

// A schedule entry of a batched build may name the one group of observations it serves: bits 8.. of `gemm` hold
// group + 1, or 0 for "every group in turn".  Returns the range of groups, strips the fields, and returns the entry's
// lag: with the two-stream schedule a CTA's list describes one CYCLE, in which the entries of stream B's gate/up and
// down phases belong to the layer pass before the cycle's (lag 1), and there is one cycle more than layer passes.
__device__ __forceinline__ int unit_groups(const Params& p, Unit& un, int& g0, int& g1) {
  if (!PI05_BATCHED) { g0 = 0; g1 = 1; return 0; }
  const int g = un.gemm >> 8, lag = (un.gemm >> 7) & 1;
  un.gemm &= 0x7f;
  if (g == 0) { g0 = 0; g1 = PI05_NGRP(p); } else { g0 = g - 1; g1 = g; }
  return lag;
}
#define PI05_CYCLES(p, npass) ((npass) + ((PI05_BATCHED && (p).stream_split > 0) ? 1 : 0))

__device__ __forceinline__ ObsPtrs obs(const Params& p, int b) {
  ObsPtrs o = p.ob;
  if (!PI05_BATCHED) return o;
  o.noise += (size_t)b * T * ADIM; o.actions += (size_t)b * T * ADIM; o.x += (size_t)b * T * ADIM;
  o.prefix_mask += (size_t)b * p.prefix;
  o.o_acc += (size_t)b * T * W; o.d_acc += (size_t)b * T * W; o.qkv_acc += (size_t)b * T * QKVW;
  o.rope += (size_t)b * T * (HD / 2); o.rope2 += (size_t)b * T * (HD / 2);
  o.h += (size_t)b * T * W; o.an_attn += (size_t)b * AN_COPIES * T * W; o.an_ffn += (size_t)b * AN_COPIES * T * W;
  o.k += (size_t)b * T * HD; o.v += (size_t)b * T * HD; o.attn += (size_t)b * T * QD; o.act += (size_t)b * T * FF;
  o.b = b;
  return o;
}

// ------------------------------------------------------------------------------------------- bounded waits
struct Ctx {
  unsigned int* status;
  long long limit;
  int cta;
  unsigned poll_ns;
};

__device__ __noinline__ void report_timeout(const Ctx& c, int kind, int stage) {
  if (atomicCAS(c.status, 0u, (unsigned)kind) == 0u) {
    c.status[1] = ((unsigned)c.cta << 16) | ((unsigned)stage & 0xffffu);
    __threadfence();
  }
}

// Returns false when the wait gave up (limit reached, or another wait already reported an error).
__device__ __forceinline__ bool wait_mbar(const Ctx& c, uint32_t bar, uint32_t parity, int kind, int stage) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned i = 0;; ++i) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 31u) {
      if (ptx::ld_relaxed(c.status) != 0u) return false;
      if (clock64() - t0 > c.limit) { report_timeout(c, kind, stage); return false; }
    }
  }
}

#if PI05_TP
// The same wait on a counter that other GPUs bump.
__device__ __forceinline__ bool wait_event_sys(const Ctx& c, const unsigned int* ev, unsigned int target, int stage) {
  if ((int)(ptx::ld_acquire_sys(ev) - target) >= 0) return true;
  const long long t0 = clock64();
  for (unsigned i = 0;; ++i) {
    if ((int)(ptx::ld_acquire_sys(ev) - target) >= 0) return true;
    if ((i & 31u) == 31u) {
      if (ptx::ld_relaxed(c.status) != 0u) return false;
      if (clock64() - t0 > c.limit) { report_timeout(c, WAIT_EVENT, stage); return false; }
    }
    __nanosleep(c.poll_ns);
  }
}
#endif

__device__ __forceinline__ bool wait_event(const Ctx& c, const unsigned int* ev, unsigned int target, int stage) {
  // One load in flight at a time on purpose: sampling the counter more often (several relaxed loads in flight)
  // was measured slower, the extra reads of the line delay the producers' updates of it.
  if ((int)(ptx::ld_acquire(ev) - target) >= 0) return true;
  const long long t0 = clock64();
  for (unsigned i = 0;; ++i) {
    if ((int)(ptx::ld_acquire(ev) - target) >= 0) return true;
    if ((i & 31u) == 31u) {
      if (ptx::ld_relaxed(c.status) != 0u) return false;
      if (clock64() - t0 > c.limit) { report_timeout(c, WAIT_EVENT, stage); return false; }
    }
    __nanosleep(c.poll_ns);
  }
}

// Called by one thread after the CTA-level barrier that follows the CTA's writes.
__device__ __forceinline__ void signal_event(unsigned int* ev) {
  ptx::red_release_add(ev, 1u);   // release at device scope: cumulative over the writes ordered by the CTA barrier
}

__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Optional in-kernel trace: GEMM CTAs 0 (gate/up), 64 (QKV) and 84 (O, down) stamp the second layer pass.
// slot = 64 + 64 * which + gemm * 8 + point; points: 0 inputs seen, 1 last act load issued, 2 first operands
// in smem, 3 all MMAs issued, 4 accumulator ready, 5 accumulator in registers, 6 stores issued, 7 signalled.
__device__ __forceinline__ void trace(const Params& p, int cta, int pass, int gemm, int point) {
  if (!PI05_TRACE || p.stamps == nullptr || pass != 1) return;
  const int which = cta == 0 ? 0 : cta == 64 ? 1 : cta == 84 ? 2 : -1;
  if (which < 0) return;
  unsigned long long* slot = p.stamps + 64 + 64 * which + gemm * 8 + point;
  if (*slot == 0) *slot = globaltimer();
}

// ------------------------------------------------------------------------------------------- small math
__device__ __forceinline__ float rb(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float gelu_tanh(float x) {
  const float z = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(z));
}

// A wait that ignores the status word: used only while leaving, for copies that are already in flight.
__device__ __forceinline__ void drain_mbar(uint32_t bar, uint32_t parity, long long limit) {
  const long long t0 = clock64();
  while (!ptx::mbar_try_wait(bar, parity))
    if (clock64() - t0 > limit) return;
}

// ------------------------------------------------------------------------------------------- prologue
// Sum ten per-lane partials over the 32 lanes with 12 shuffles, for R independent rows at once (the rows give the
// scheduler independent shuffle chains to overlap).  Lanes with an even index end up holding in v[r][0] the total
// of value `idx` of row r (idx < 0: nothing).  The order of additions is fixed.
template <int R>
__device__ __forceinline__ int reduce10(float (&v)[R][10], int lane) {
  const unsigned full = 0xffffffffu;
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
#pragma unroll
  for (int i = 0; i < 5; ++i)
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float send = b4 ? v[r][i] : v[r][i + 5];
      const float keep = b4 ? v[r][i + 5] : v[r][i];
      v[r][i] = keep + __shfl_xor_sync(full, send, 16);
    }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float s0 = b3 ? v[r][0] : v[r][3], k0 = b3 ? v[r][3] : v[r][0];
    const float s1 = b3 ? v[r][1] : v[r][4], k1 = b3 ? v[r][4] : v[r][1];
    const float s2 = b3 ? v[r][2] : 0.f, k2 = b3 ? 0.f : v[r][2];
    v[r][0] = k0 + __shfl_xor_sync(full, s0, 8);
    v[r][1] = k1 + __shfl_xor_sync(full, s1, 8);
    v[r][2] = k2 + __shfl_xor_sync(full, s2, 8);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float s0 = b2 ? v[r][0] : v[r][2], k0 = b2 ? v[r][2] : v[r][0];
    const float s1 = b2 ? v[r][1] : 0.f, k1 = b2 ? 0.f : v[r][1];
    v[r][0] = k0 + __shfl_xor_sync(full, s0, 4);
    v[r][1] = k1 + __shfl_xor_sync(full, s1, 4);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float s0 = b1 ? v[r][0] : v[r][1], k0 = b1 ? v[r][1] : v[r][0];
    v[r][0] = k0 + __shfl_xor_sync(full, s0, 2);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) v[r][0] += __shfl_xor_sync(full, v[r][0], 1);
  const int in5 = b3 ? (b2 ? -1 : 3 + (b1 ? 1 : 0)) : (b2 ? (b1 ? -1 : 2) : (b1 ? 1 : 0));
  return in5 < 0 ? -1 : in5 + (b4 ? 5 : 0);
}

// out[s][row] = f(W[row][:] . in[s][:] + bias[row]) for the ten time steps at once; FP32 weights streamed from
// HBM exactly once.  Four warps share a row (a quarter of K each, the ten input vectors of that quarter live in
// registers), four rows per batch, and the loads of the next batch are issued before the current one is reduced, so
// every warp keeps 4-8 KB in flight.  MODE 0/1: time MLP layers (SiLU).  MODE 2: the 37 modulation layers.
template <int MODE>
__device__ void matvec10(const Params& p, const float* __restrict__ in, uint8_t* smem, int cta, int ncta) {
  constexpr int RB = 4;                      // rows per batch
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp >> 2, quarter = warp & 3;
  const int koff = quarter * 256 + lane * 4;
  float c[NS][8];
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    const float4 a = *reinterpret_cast<const float4*>(in + s * W + koff);
    const float4 b = *reinterpret_cast<const float4*>(in + s * W + koff + 128);
    c[s][0] = a.x; c[s][1] = a.y; c[s][2] = a.z; c[s][3] = a.w;
    c[s][4] = b.x; c[s][5] = b.y; c[s][6] = b.z; c[s][7] = b.w;
  }
  float* part = reinterpret_cast<float*>(smem + OFF_STAGE);  // [2 buf][2 group][4 quarter][RB row][10]
  const int nrows = (MODE == 2) ? NNORM * MODW : W;
  const int nbatch = nrows / RB;
  const int stride = ncta * 2;

  auto weight_base = [&](int row0) -> const float* {
    if (MODE == 0) return p.tin_w + (size_t)row0 * W;
    if (MODE == 1) return p.tout_w + (size_t)row0 * W;
    const int n = row0 / MODW, j = row0 % MODW;
    if (n == NNORM - 1) return p.fin_nw + (size_t)j * W;
    return ((n & 1) ? p.ffn_nw : p.attn_nw) + ((size_t)(n >> 1) * MODW + j) * W;
  };
  auto load = [&](float4 (&w)[RB][2], int b) {
    const float* wbase = weight_base(b * RB) + koff;
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      w[r][0] = ptx::ldg_stream_f4(wbase + (size_t)r * W);
      w[r][1] = ptx::ldg_stream_f4(wbase + (size_t)r * W + 128);
    }
  };
  auto reduce_store = [&](const float4 (&w)[RB][2], int b, int it) {
    // the bias of the output this thread will write is fetched first, so that its latency hides behind the FMAs
    const int i = tid & 127, orow = b * RB + i / 10, os = i % 10;
    float bias = 0.f;
    float* out = nullptr;
    if (i < RB * 10) {
      if (MODE == 0) { bias = p.tin_b[orow]; out = p.hid + (size_t)os * W + orow; }
      else if (MODE == 1) { bias = p.tout_b[orow]; out = p.cond + (size_t)os * W + orow; }
      else {
        const int n = orow / MODW, j = orow % MODW;
        bias = n == NNORM - 1 ? p.fin_nb[j] : ((n & 1) ? p.ffn_nb : p.attn_nb)[(size_t)(n >> 1) * MODW + j];
        out = p.mod + ((size_t)os * NNORM + n) * MODW + j;
      }
    }
    float* pb = part + (((it & 1) * 2 + group) * 4 + quarter) * (RB * 10);
    float acc[RB][10];
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        float a = w[r][0].x * c[s][0];
        a = fmaf(w[r][0].y, c[s][1], a);
        a = fmaf(w[r][0].z, c[s][2], a);
        a = fmaf(w[r][0].w, c[s][3], a);
        a = fmaf(w[r][1].x, c[s][4], a);
        a = fmaf(w[r][1].y, c[s][5], a);
        a = fmaf(w[r][1].z, c[s][6], a);
        a = fmaf(w[r][1].w, c[s][7], a);
        acc[r][s] = a;
      }
    const int idx = reduce10<RB>(acc, lane);
    if (!(lane & 1) && idx >= 0) {
#pragma unroll
      for (int r = 0; r < RB; ++r) pb[r * 10 + idx] = acc[r][0];
    }
    ptx::named_bar_sync(2 + group, 128);
    if (i < RB * 10) {
      const float* q0 = part + (((it & 1) * 2 + group) * 4) * (RB * 10) + i;
      const float v = ((q0[0] + q0[RB * 10]) + (q0[2 * RB * 10] + q0[3 * RB * 10])) + bias;
      *out = (MODE == 2) ? v : silu(v);
    }
  };

  float4 wa[RB][2], wb[RB][2];
  int b = cta * 2 + group, it = 0;
  if (b < nbatch) load(wa, b);
  while (b < nbatch) {
    const int b1 = b + stride;
    if (b1 < nbatch) load(wb, b1);
    reduce_store(wa, b, it++);
    if (b1 >= nbatch) break;
    const int b2 = b1 + stride;
    if (b2 < nbatch) load(wa, b2);
    reduce_store(wb, b1, it++);
    b = b2;
  }
}

// Grid-wide rendezvous of the prologue: every CTA arrives, every CTA waits.
__device__ bool grid_event(const Params& p, const Ctx& c, int ev, int ncta) {
  __syncthreads();
  __shared__ int ok_flag;
  if (threadIdx.x == 0) {
    signal_event(p.ctrl + EVW(ev));
    ok_flag = wait_event(c, p.ctrl + EVW(ev), (unsigned)ncta, -1 - ev) ? 1 : 0;
  }
  __syncthreads();
  return ok_flag != 0;
}

__device__ int count_valid(const Params& p, const ObsPtrs& o) {
  __shared__ int s_cnt;
  __syncthreads();
  if (threadIdx.x == 0) s_cnt = 0;
  __syncthreads();
  int n = 0;
  for (int i = threadIdx.x; i < p.prefix; i += THREADS) n += o.prefix_mask[i] ? 1 : 0;
  for (int sh = 16; sh; sh >>= 1) n += __shfl_xor_sync(0xffffffffu, n, sh);
  if ((threadIdx.x & 31) == 0 && n) atomicAdd(&s_cnt, n);
  __syncthreads();
  return s_cnt;
}

// Time embedding (FP64, reference/pi05.py:232-237), and per observation the RoPE tables (reference/pi05.py:218-229;
// positions start at that observation's number of valid prefix tokens) and the clearing of its split-K accumulators.
__device__ void prologue_tables(const Params& p, int cta, int ncta) {
  const int gtid = cta * THREADS + threadIdx.x, gn = ncta * THREADS;
  for (int i = gtid; i < NS * W; i += gn) {
    const int s = i / W, j = i % W, f = j % (W / 2);
    const double step = 1.0 / (W / 2 - 1);
    const double frac = f < (W / 4) ? step * f : 1.0 - step * (W / 2 - 1 - f);
    const double period = 4e-3 * pow(4.0 / 4e-3, frac);
    const double phase = (double)p.t_steps[s] * (1.0 / period * 2 * 3.141592653589793);
    p.temb[i] = (float)(j < W / 2 ? sin(phase) : cos(phase));
  }
  for (int b = 0; b < PI05_NB(p); ++b) {
    const ObsPtrs o = obs(p, b);
    const int nvalid = count_valid(p, o);
    for (int i = gtid; i < T * (HD / 2); i += gn) {
      const int t = i / (HD / 2), j = i % (HD / 2);
      const float e = (float)(2 * j) / (float)HD;
      const float inv = 1.0f / (float)pow(10000.0, (double)e);
      const float phase = (float)(nvalid + t) * inv;
      o.rope[i] = pack_bf16((float)cos((double)phase), (float)sin((double)phase));
    }
    for (int i = gtid; i < (T / 2) * (HD / 2); i += gn) {
      const int tp = i / (HD / 2), j = i % (HD / 2);
      const float e = (float)(2 * j) / (float)HD;
      const float inv = 1.0f / (float)pow(10000.0, (double)e);
      const float ph0 = (float)(nvalid + 2 * tp) * inv, ph1 = (float)(nvalid + 2 * tp + 1) * inv;
      o.rope2[2 * i] = pack_bf16((float)cos((double)ph0), (float)cos((double)ph1));
      o.rope2[2 * i + 1] = pack_bf16((float)sin((double)ph0), (float)sin((double)ph1));
    }
    for (int i = gtid; i < T * QKVW; i += gn) o.qkv_acc[i] = 0.f;
    for (int i = gtid; i < T * W; i += gn) { o.o_acc[i] = 0.f; o.d_acc[i] = 0.f; }
  }
}

// ------------------------------------------------------------------------------------------- row operations
enum { ROW_INIT = 0, ROW_ATT = 1, ROW_FFN = 2 };

// Modulation values a row operation needs; they depend only on the step and the layer, so they are fetched
// before the wait for the GEMM that feeds the operation.
struct RowMod { float gate[8], scale[8], shift[8]; };

__device__ __forceinline__ void row_prefetch(const Params& p, int mode, int step, int layer, RowMod& rm) {
  const int c0 = (threadIdx.x & 127) * 8;
  const float* mod_s = p.mod + (size_t)step * NNORM * MODW;
  int gate_norm, next_norm;
  if (mode == ROW_ATT) { gate_norm = 2 * layer; next_norm = 2 * layer + 1; }
  else { gate_norm = 2 * layer + 1; next_norm = (layer + 1 < p.n_layers) ? 2 * layer + 2 : NNORM - 1; }
  const float* g = mod_s + (size_t)gate_norm * MODW + 2 * W + c0;
  const float* n = mod_s + (size_t)next_norm * MODW + c0;
#pragma unroll
  for (int e = 0; e < 8; e += 4) {
    const float4 a = *reinterpret_cast<const float4*>(g + e), b = *reinterpret_cast<const float4*>(n + e),
                 d = *reinterpret_cast<const float4*>(n + W + e);
    rm.gate[e] = a.x; rm.gate[e + 1] = a.y; rm.gate[e + 2] = a.z; rm.gate[e + 3] = a.w;
    rm.scale[e] = b.x; rm.scale[e + 1] = b.y; rm.scale[e + 2] = b.z; rm.scale[e + 3] = b.w;
    rm.shift[e] = d.x; rm.shift[e + 1] = d.y; rm.shift[e + 2] = d.z; rm.shift[e + 3] = d.w;
  }
}

// Per-token work between GEMMs, two tokens per CTA, 128 threads per token, 8 columns per thread.  The thread
// keeps its 8 values of the residual stream h in registers (hn) from one call to the next.
//   ROW_ATT: h += bf16(bf16(o_acc) * gate_attn); an_ffn = adaRMS_ffn(h)
//   ROW_FFN: h += bf16(bf16(d_acc) * gate_ffn); then either an_attn = adaRMS_attn[l+1](h), or at the last layer
//            the step tail: final adaRMS, v = Wout n + b, x += dt v, and (unless it was the last step)
//            h = bf16(Win x + b), an_attn = adaRMS_attn[0](h) with the next step's modulation.
//   ROW_INIT: x = noise, h = bf16(Win x + b), an_attn = adaRMS_attn[0](h).
// Tensor parallel: the accumulator then holds only this rank's share of the sum (its heads, its MLP columns).  Every
// rank stores its two rows into its slot of every peer's receive buffer, bumps the peer's counter for this row CTA
// (release at system scope, after a CTA barrier), waits until all peers have done the same here, and adds the
// size partial sums in rank order - the same order on every rank, so every rank keeps the same residual stream.
// Returns false when that wait gave up.
__device__ bool row_op(const Params& p, const Ctx& c, const ObsPtrs& o, uint8_t* smem, int unit, int mode, int step, int layer,
                       int pass, float (&hn)[8], const RowMod& rm) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int half = tid >> 7, i = tid & 127, wq = (tid >> 5) & 3;
  const int t = unit * 2 + half;
  const int c0 = i * 8;
  float* rowbuf = reinterpret_cast<float*>(smem + OFF_ROWBUF) + half * (1024 + 64);
  float* red = rowbuf + 1024;      // [0..3] warp sums, [8..39] x row
  const int bar = 4 + half;

  auto sumsq = [&](const float (&v)[8]) -> float {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    for (int sh = 16; sh; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
    ptx::named_bar_sync(bar, 128);          // previous use of red[] is over
    if (lane == 0) red[wq] = ss;
    ptx::named_bar_sync(bar, 128);
    return (red[0] + red[1]) + (red[2] + red[3]);
  };
  auto ada_norm = [&](const float (&v)[8], const float (&scale)[8], const float (&shift)[8], __nv_bfloat16* dst) {
    const float ss = sumsq(v);
    const float rs = 1.0f / sqrtf(ss * (1.0f / W) + EPS);
    uint32_t ow[4];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const float a = __fadd_rn(__fmul_rn(__fmul_rn(v[e], rs), __fadd_rn(1.0f, scale[e])), shift[e]);
      const float b = __fadd_rn(__fmul_rn(__fmul_rn(v[e + 1], rs), __fadd_rn(1.0f, scale[e + 1])), shift[e + 1]);
      ow[e >> 1] = pack_bf16(a, b);
    }
#pragma unroll
    for (int r = 0; r < AN_COPIES; ++r)   // one copy per group of reader CTAs
      *reinterpret_cast<uint4*>(dst + ((size_t)r * T + t) * W + c0) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  };
  auto store_h = [&](const float (&v)[8]) {   // the kernel itself never reads h back; kept for stage-level checks
    const uint4 packed = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
    *reinterpret_cast<uint4*>(o.h + (size_t)t * W + c0) = packed;
  };
  // h = bf16(Win x + b) for this thread's 8 columns; x row in red[8..39]
  auto action_in = [&]() {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float* wr = p.ain_w + (size_t)(c0 + e) * ADIM;
      float a = 0.f;
#pragma unroll
      for (int k = 0; k < ADIM; k += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(wr + k);
        a = fmaf(w4.x, red[8 + k], a); a = fmaf(w4.y, red[9 + k], a);
        a = fmaf(w4.z, red[10 + k], a); a = fmaf(w4.w, red[11 + k], a);
      }
      hn[e] = rb(a + p.ain_b[c0 + e]);
    }
  };
  auto next_step_norm = [&](int s) {          // attention norm of layer 0 with the modulation of step s
    const float* m = p.mod + (size_t)s * NNORM * MODW + c0;
    float sc[8], sh[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { sc[e] = m[e]; sh[e] = m[W + e]; }
    ada_norm(hn, sc, sh, o.an_attn);
  };

  if (mode == ROW_INIT) {
    if (i < ADIM) { const float xv = o.noise[t * ADIM + i]; o.x[t * ADIM + i] = xv; red[8 + i] = xv; }
    ptx::named_bar_sync(bar, 128);
    action_in();
    store_h(hn);
    next_step_norm(0);
    return true;
  }

  // gated residual.  With a batch of one the residual stream stays in this thread's registers between row
  // operations; with more observations it is re-read from memory.
  if (PI05_NB(p) > 1) {
    const uint4 hv = *reinterpret_cast<const uint4*>(o.h + (size_t)t * W + c0);
    const uint32_t hw[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) hn[e] = (e & 1) ? bf16_hi(hw[e >> 1]) : bf16_lo(hw[e >> 1]);
  }
  float* acc = (mode == ROW_ATT ? o.o_acc : o.d_acc) + (size_t)t * W + c0;
  {
    const float4 a0 = __ldcg(reinterpret_cast<const float4*>(acc)), a1 = __ldcg(reinterpret_cast<const float4*>(acc + 4));
    *reinterpret_cast<float4*>(acc) = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(acc + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#if PI05_TP
    if (p.tp_size > 1) {
      const int kind = mode == ROW_ATT ? 0 : 1;
      const size_t at = ((size_t)(kind * p.tp_size + p.tp_rank) * T + t) * W + c0;
      for (int r = 0; r < p.tp_size; ++r)
        if (r != p.tp_rank) {
          *reinterpret_cast<float4*>(p.tp_peer_recv[r] + at) = a0;
          *reinterpret_cast<float4*>(p.tp_peer_recv[r] + at + 4) = a1;
        }
      __syncthreads();                 // every thread's stores precede the release below (cumulative over the barrier)
      __shared__ int tp_ok;
      if (tid == 0) {
        const int slot = (kind * NROW_CTAS + unit) * TP_FLAG_STRIDE;
        for (int r = 0; r < p.tp_size; ++r)
          if (r != p.tp_rank) ptx::red_release_sys_add(p.tp_peer_flags[r] + slot, 1u);
        tp_ok = wait_event_sys(c, p.tp_flags + slot, p.tp_base + (unsigned)((p.tp_size - 1) * (pass + 1)),
                               pass * NSTAGE + (kind ? ST_RFFN : ST_RATT)) ? 1 : 0;
      }
      __syncthreads();
      if (!tp_ok) return false;
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < p.tp_size; ++r) {
        float pv[8];
        if (r == p.tp_rank) {
#pragma unroll
          for (int e = 0; e < 8; ++e) pv[e] = av[e];
        } else {
          const float* src = p.tp_recv + ((size_t)(kind * p.tp_size + r) * T + t) * W + c0;
          const float4 b0 = __ldcg(reinterpret_cast<const float4*>(src)), b1 = __ldcg(reinterpret_cast<const float4*>(src + 4));
          pv[0] = b0.x; pv[1] = b0.y; pv[2] = b0.z; pv[3] = b0.w; pv[4] = b1.x; pv[5] = b1.y; pv[6] = b1.z; pv[7] = b1.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sum[e] += pv[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) av[e] = sum[e];
    }
#endif
#pragma unroll
    for (int e = 0; e < 8; ++e) hn[e] = rb(hn[e] + rb(rb(av[e]) * rb(rm.gate[e])));
  }
  store_h(hn);
  if (mode == ROW_ATT) {
    float4* z = reinterpret_cast<float4*>(o.qkv_acc + (size_t)t * QKVW) + i;
#pragma unroll
    for (int e = 0; e < QKVW / 4 / 128; ++e) z[e * 128] = make_float4(0.f, 0.f, 0.f, 0.f);
    ada_norm(hn, rm.scale, rm.shift, o.an_ffn);
    return true;
  }
  if (layer + 1 < p.n_layers) { ada_norm(hn, rm.scale, rm.shift, o.an_attn); return true; }
  // ---- step tail: final norm, action_out, Euler update
  {
    const float ss = sumsq(hn);
    const float rs = 1.0f / sqrtf(ss * (1.0f / W) + EPS);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      rowbuf[c0 + e] = rb(__fadd_rn(__fmul_rn(__fmul_rn(hn[e], rs), __fadd_rn(1.0f, rm.scale[e])), rm.shift[e]));
    ptx::named_bar_sync(bar, 128);
    // warp wq: outputs wq*8 .. wq*8+7
    for (int a = wq * 8; a < wq * 8 + 8; ++a) {
      const float* wr = p.aout_w + (size_t)a * W;
      float sdot = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = lane * 4 + j * 128;
        const float4 w4 = *reinterpret_cast<const float4*>(wr + k);
        sdot = fmaf(w4.x, rowbuf[k], sdot); sdot = fmaf(w4.y, rowbuf[k + 1], sdot);
        sdot = fmaf(w4.z, rowbuf[k + 2], sdot); sdot = fmaf(w4.w, rowbuf[k + 3], sdot);
      }
      for (int sh = 16; sh; sh >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, sh);
      if (lane == 0) {
        const float vel = sdot + p.aout_b[a];
        const float xn = __fadd_rn(o.x[t * ADIM + a], __fmul_rn(p.dt, vel));
        o.x[t * ADIM + a] = xn;
        red[8 + a] = xn;
        if (step + 1 == p.n_steps) o.actions[t * ADIM + a] = xn;
      }
    }
    ptx::named_bar_sync(bar, 128);
    if (step + 1 < p.n_steps) {
      action_in();
      store_h(hn);
      next_step_norm(step + 1);
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------------- attention
// 16 query rows (2 tokens x 8 heads, all sharing the one KV head) against [prefix ; suffix] keys.  Keys are
// staged in shared memory in 64-key chunks, three chunks (192 keys) at a time; with a prefix of 128 that is
// everything, in one pass.  Scores: bf16(q.k) / 16, masked; running max; p = bf16(exp(s - m)); o += p V (FP32);
// out = bf16(o / sum exp).
// q leaves the QKV GEMM as FP32 split-K sums.  The row CTA finishes its 16 query rows while staging them: round to
// BF16 (the GEMM's output rounding), then RoPE with every product and the sum rounded to BF16
// (reference/pi05.py:218-229: x * cos + rotate_half(x) * sin on BF16 tensors).  One item of 8 rotary pairs per thread.
__device__ void build_q(const ObsPtrs& o, uint8_t* smem, int unit) {
  const int tid = threadIdx.x;
  const int m = tid >> 4, d0 = (tid & 15) * 8, t = unit * 2 + (m >> 3);
  const float* lo = o.qkv_acc + (size_t)t * QKVW + (m & 7) * HD + d0;
  const uint32_t* cs = o.rope + t * (HD / 2) + d0;
  const float4 x0 = __ldcg(reinterpret_cast<const float4*>(lo)), x1 = __ldcg(reinterpret_cast<const float4*>(lo + 4));
  const float4 y0 = __ldcg(reinterpret_cast<const float4*>(lo + 128)), y1 = __ldcg(reinterpret_cast<const float4*>(lo + 132));
  const uint4 c0 = __ldcg(reinterpret_cast<const uint4*>(cs)), c1 = __ldcg(reinterpret_cast<const uint4*>(cs + 4));
  const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
  const float y[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
  const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  float o1[8], o2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float xb = rb(x[i]), yb = rb(y[i]), co = bf16_lo(cw[i]), si = bf16_hi(cw[i]);
    o1[i] = rb(xb * co) + rb(-yb * si);     // rotate_half: first half x*cos - y*sin
    o2[i] = rb(yb * co) + rb(xb * si);      // second half y*cos + x*sin
  }
  const uint32_t dst = ptx::smem_u32(smem + OFF_QS) + (m * KV_STRIDE + d0) * 2;
  ptx::st_shared_v4(dst, pack_bf16(o1[0], o1[1]), pack_bf16(o1[2], o1[3]), pack_bf16(o1[4], o1[5]), pack_bf16(o1[6], o1[7]));
  ptx::st_shared_v4(dst + 256, pack_bf16(o2[0], o2[1]), pack_bf16(o2[2], o2[3]), pack_bf16(o2[4], o2[5]), pack_bf16(o2[6], o2[7]));
}

__device__ bool cta_wait_event(const Params& p, const Ctx& c, int word, unsigned target, int stage) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = wait_event(c, p.ctrl + word, target, stage) ? 1 : 0;
  __syncthreads();
  const int ok = ok_flag;
  __syncthreads();
  return ok != 0;
}

// Parities of the attention barriers of a row CTA (bit j: keys of stage j, bit 8 + j: values of stage j) and which of
// them have a copy in flight that nobody has waited for yet.
struct AttBars {
  uint32_t parity = 0, pending = 0;
};

__device__ __forceinline__ uint32_t att_bar(uint8_t* smem, int isv, int stage) {
  return ptx::smem_u32(smem + OFF_ATTBARS) + 8 * (isv * ATT_STAGES + stage);
}

// All threads wait until the keys (isv = 0) or values (isv = 1) of `stage` have landed.
__device__ __forceinline__ bool att_wait(const Ctx& c, uint8_t* smem, AttBars& bars, int isv, int stage, int st) {
  const uint32_t bit = 1u << (8 * isv + stage);
  const bool ok = wait_mbar(c, att_bar(smem, isv, stage), (bars.parity & bit) ? 1u : 0u, WAIT_A_FULL, st);
  bars.parity ^= bit;
  bars.pending &= ~bit;
  return ok;
}

// Before a row CTA gives up: let its own copies in flight land (bounded like every wait).
__device__ void att_drain(const Ctx& c, uint8_t* smem, AttBars& bars, int st) {
  for (int isv = 0; isv < 2; ++isv)
    for (int j = 0; j < ATT_STAGES; ++j)
      if (bars.pending & (1u << (8 * isv + j))) att_wait(c, smem, bars, isv, j, st);
}

struct AttChunkIssue {
  const Params& p;
  const ObsPtrs& o;
  const Ctx& c;
  uint8_t* smem;
  AttBars& bars;
  int layer, npc, pass, cend;
  // chunk < npc: prefix keys [64*chunk, ...); chunk == npc: the 50 suffix keys; chunk >= cend (the end of this CTA's
  // share of the keys) or > npc: nothing (stage off)
  // `which`: 1 = keys only, 2 = values (and the validity bytes, which the previous occupant's softmax has read by
  // then) only, 3 = both.  One thread issues one tiled copy per chunk of keys or of values (four 64-dim segments); it
  // completes on the stage's barrier, and rows past the end of a short chunk arrive as zeros.
  // Collective over the CTA.  Returns false when the wait for the suffix keys gave up.
  __device__ bool operator()(int chunk, int stage, int which = 3) const {
    const int tid = threadIdx.x;
    const bool live = chunk <= npc && chunk < cend;
    if (chunk == npc && live && (which & 1) &&
        !cta_wait_event(p, c, EVB(EV_KV, o.b), NKVTILES * (pass + 1), pass * NSTAGE + ST_ATT)) return false;
    const bool is_prefix = chunk < npc;
    if (tid < 64 && (which & 2)) {
      const int nrows = !live ? 0 : (is_prefix ? min(64, p.prefix - chunk * 64) : T);
      uint8_t ok = 0;
      if (tid < nrows) ok = is_prefix ? (o.prefix_mask[chunk * 64 + tid] ? 1 : 0) : 1;
      smem[OFF_KVALID + stage * 64 + tid] = ok;
    }
    if (!live) return true;
#pragma unroll
    for (int isv = 0; isv < 2; ++isv) {
      if (!((which >> isv) & 1)) continue;
      if (tid == 0) {
        const uint32_t dst = ptx::smem_u32(smem + (isv ? OFF_VS : OFF_KS) + stage * KV_STAGE_BYTES);
        const uint32_t bar = att_bar(smem, isv, stage);
        ptx::mbar_expect_tx(bar, KV_STAGE_BYTES);
        if (is_prefix) {
          // logical page of the chunk -> physical page of the pool; the last page goes through the map whose rows
          // end at the last valid token, so that whatever lies behind it in the cache arrives as zeros
          const int lp = p.pages_per_obs == 1 ? 0 : chunk * 64 / p.page_tokens, row = chunk * 64 - lp * p.page_tokens;
          const int phys = reinterpret_cast<const int*>(smem + OFF_PAGETAB)[o.b * p.pages_per_obs + lp];
          const bool tail = lp == (p.prefix - 1) / p.page_tokens;
          const CUtensorMap* m = tail ? (isv ? &p.maps.pv_tail : &p.maps.pk_tail) : (isv ? &p.maps.pv : &p.maps.pk);
          ptx::tma_load_5d(dst, m, bar, 0, row, 0, layer, phys);
        } else {
          ptx::fence_proxy_async_global();   // the suffix rows were written by GEMM epilogues
          ptx::tma_load_4d(dst, isv ? &p.maps.sv : &p.maps.sk, bar, 0, 0, 0, o.b);
        }
      }
      bars.pending |= 1u << (8 * isv + stage);
    }
    return true;
  }
};

constexpr int QF_KEPT = PI05_QF_KEPT;   // 16-dim blocks of q (of 16) whose A fragments stay in registers (even)
// S = Q K^T for this warp's 8 keys of one stage (two interleaved accumulation chains).
__device__ __forceinline__ void att_qk(const uint32_t (&qf)[QF_KEPT][4], uint32_t qs, uint32_t ks, int warp, int lane,
                                       float (&s4)[4]) {
  const uint32_t qaddr0 = qs + ((lane & 15) * KV_STRIDE + (lane >> 4) * 8) * 2;
  float e[4] = {0.f, 0.f, 0.f, 0.f}, o[4] = {0.f, 0.f, 0.f, 0.f};
  // key row r = warp * 8 + (lane & 7); 16-byte piece c of the row sits at piece c ^ (r & 7) of its 128-byte line
  const uint32_t krow = ks + (warp * 8 + (lane & 7)) * 128;
  const uint32_t ksw = lane & 7, kc = lane >> 3;
#pragma unroll
  for (int kk = 0; kk < HD / 16; kk += 2) {
    uint32_t b0, b1, b2, b3;
    ptx::ldmatrix_x4(krow + (kk >> 2) * KV_SEG_BYTES + ((((kk & 3) * 2 + kc) ^ ksw) << 4), b0, b1, b2, b3);
    if (kk < QF_KEPT) {      // the first blocks of q stay in registers, the rest is fetched again for every stage
      ptx::mma_16816(e, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
      ptx::mma_16816(o, qf[kk + 1][0], qf[kk + 1][1], qf[kk + 1][2], qf[kk + 1][3], b2, b3);
    } else {
      uint32_t a0, a1, a2, a3, a4, a5, a6, a7;
      ptx::ldmatrix_x4(qaddr0 + kk * 32, a0, a1, a2, a3);
      ptx::ldmatrix_x4(qaddr0 + kk * 32 + 32, a4, a5, a6, a7);
      ptx::mma_16816(e, a0, a1, a2, a3, b0, b1);
      ptx::mma_16816(o, a4, a5, a6, a7, b2, b3);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) s4[i] = e[i] + o[i];
}

// The first `nearly` stages (prefix chunks) were issued by the caller before q was ready.  Scores against them are
// computed first; the suffix keys are waited for and copied only then, so the k / v tiles of the QKV GEMM may
// finish later than the q tiles without holding attention up.  Returns false when a wait gave up.
// With key groups (one observation, long prefix) the CTA covers only chunks [cbeg, cend) of the keys: groups >= 1 leave
// their unnormalised accumulators, running maxima and sums in global memory (`kg` = their group), group 0 merges
// them into its own (flash-decoding style) before it normalises.
__device__ bool attention_unit(const Params& p, const ObsPtrs& o, uint8_t* smem, int unit, const AttChunkIssue& issue,
                               int cbeg, int nearly, int kg, bool tr) {
  const int cend = issue.cend, wst = issue.pass * NSTAGE + ST_ATT;
  AttBars& bars = issue.bars;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, qd = lane & 3;
  const uint32_t qs = ptx::smem_u32(smem + OFF_QS), ps = ptx::smem_u32(smem + OFF_PS);
  float* red = reinterpret_cast<float*>(smem + OFF_RED);
  const float NEG = -INFINITY;

  float m_lo = -1e30f, m_hi = -1e30f, l_lo = 0.f, l_hi = 0.f;
  uint32_t qf[QF_KEPT][4];
  float oa[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) oa[a][b] = 0.f;

  for (int c0 = cbeg; c0 < cend; c0 += ATT_STAGES) {
    const int nst = min(ATT_STAGES, cend - c0);
    float sc[ATT_STAGES][4];
    // ---- scores; in the first pass the prefix stages are used while the suffix keys are still being produced
    const int early = (c0 == cbeg) ? nearly : nst;
    const bool more = c0 + ATT_STAGES < cend;
    __syncthreads();                                   // q is in place (first round)
    if (c0 == cbeg) {
      // the whole 16 x 256 q tile as A fragments, kept in registers for every stage of every round
      const uint32_t qaddr0 = qs + ((lane & 15) * KV_STRIDE + (lane >> 4) * 8) * 2;
#pragma unroll
      for (int kk = 0; kk < QF_KEPT; ++kk) ptx::ldmatrix_x4(qaddr0 + kk * 32, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
    }
    if (tr && c0 == cbeg) p.stamps[224] = globaltimer();
    if (tr && c0 != cbeg && !more) p.stamps[232] = globaltimer();
#pragma unroll
    for (int j = 0; j < ATT_STAGES; ++j)
      if (j < early) {
        if (!att_wait(issue.c, smem, bars, 0, j, wst)) return false;
        att_qk(qf, qs, ptx::smem_u32(smem + OFF_KS + j * KV_STAGE_BYTES), warp, lane, sc[j]);
      }
    if (early < nst) {
      if (!issue(c0 + early, early)) return false;     // waits for the k / v tiles, then copies the suffix chunk
#pragma unroll
      for (int j = 0; j < ATT_STAGES; ++j)
        if (j >= early && j < nst) {
          if (!att_wait(issue.c, smem, bars, 0, j, wst)) return false;
          att_qk(qf, qs, ptx::smem_u32(smem + OFF_KS + j * KV_STAGE_BYTES), warp, lane, sc[j]);
        }
    }
    if (tr && c0 == cbeg) p.stamps[225] = globaltimer();
    if (tr && c0 != cbeg && !more) p.stamps[233] = globaltimer();
    // ---- mask, chunk max
    float cm_lo = NEG, cm_hi = NEG;
#pragma unroll
    for (int j = 0; j < ATT_STAGES; ++j) {
      if (j < nst) {
        const uint8_t* kvalid = smem + OFF_KVALID + j * 64 + warp * 8 + 2 * qd;
        const bool v0 = kvalid[0] != 0, v1 = kvalid[1] != 0;
        sc[j][0] = v0 ? rb(sc[j][0]) * 0.0625f : NEG; sc[j][1] = v1 ? rb(sc[j][1]) * 0.0625f : NEG;
        sc[j][2] = v0 ? rb(sc[j][2]) * 0.0625f : NEG; sc[j][3] = v1 ? rb(sc[j][3]) * 0.0625f : NEG;
        cm_lo = fmaxf(cm_lo, fmaxf(sc[j][0], sc[j][1]));
        cm_hi = fmaxf(cm_hi, fmaxf(sc[j][2], sc[j][3]));
      }
    }
    cm_lo = fmaxf(cm_lo, __shfl_xor_sync(0xffffffffu, cm_lo, 1));
    cm_lo = fmaxf(cm_lo, __shfl_xor_sync(0xffffffffu, cm_lo, 2));
    cm_hi = fmaxf(cm_hi, __shfl_xor_sync(0xffffffffu, cm_hi, 1));
    cm_hi = fmaxf(cm_hi, __shfl_xor_sync(0xffffffffu, cm_hi, 2));
    if (qd == 0) { red[warp * 16 + g] = cm_lo; red[warp * 16 + g + 8] = cm_hi; }
    __syncthreads();
    float mn_lo = m_lo, mn_hi = m_hi;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) {
      mn_lo = fmaxf(mn_lo, red[w8 * 16 + g]);
      mn_hi = fmaxf(mn_hi, red[w8 * 16 + g + 8]);
    }
    // every warp has scored these key stages: refill them for the next round while softmax and P V run
    if (more) {
      for (int j = 0; j < ATT_STAGES; ++j)
        if (!issue(c0 + ATT_STAGES + j, j, 1)) return false;
    }
    const float al_lo = __expf(m_lo - mn_lo), al_hi = __expf(m_hi - mn_hi);
    m_lo = mn_lo; m_hi = mn_hi;
    l_lo *= al_lo; l_hi *= al_hi;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { oa[nt][0] *= al_lo; oa[nt][1] *= al_lo; oa[nt][2] *= al_hi; oa[nt][3] *= al_hi; }
#pragma unroll
    for (int j = 0; j < ATT_STAGES; ++j) {
      if (j < nst) {
        const float p00 = __expf(sc[j][0] - mn_lo), p01 = __expf(sc[j][1] - mn_lo);
        const float p10 = __expf(sc[j][2] - mn_hi), p11 = __expf(sc[j][3] - mn_hi);
        l_lo += p00 + p01;
        l_hi += p10 + p11;
        uint8_t* pbase = smem + OFF_PS + (j * 64 + warp * 8 + 2 * qd) * 2;
        *reinterpret_cast<uint32_t*>(pbase + g * P_STRIDE * 2) = pack_bf16(p00, p01);
        *reinterpret_cast<uint32_t*>(pbase + (g + 8) * P_STRIDE * 2) = pack_bf16(p10, p11);
      }
    }
    __syncthreads();
    if (tr && c0 == cbeg) p.stamps[226] = globaltimer();
    if (tr && c0 != cbeg && !more) p.stamps[234] = globaltimer();
    // ---- O += P V for this warp's 32 output dims
#pragma unroll
    for (int j = 0; j < ATT_STAGES; ++j) {
      if (j < nst) {
        if (!att_wait(issue.c, smem, bars, 1, j, wst)) return false;
        const uint32_t vs = ptx::smem_u32(smem + OFF_VS + j * KV_STAGE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          uint32_t a0, a1, a2, a3, r0, r1, r2, r3, r4, r5, r6, r7;
          ptx::ldmatrix_x4(ps + ((lane & 15) * P_STRIDE + j * 64 + kk * 16 + (lane >> 4) * 8) * 2, a0, a1, a2, a3);
          // value row r, dims db + (lane >> 4) * 8 (+16): segment warp / 2, piece (warp & 1) * 4 + (lane >> 4) (+2)
          const uint32_t vrow = vs + (warp >> 1) * KV_SEG_BYTES + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * 128;
          const uint32_t vc = (warp & 1) * 4 + (lane >> 4), vsw = lane & 7;
          ptx::ldmatrix_x4_trans(vrow + ((vc ^ vsw) << 4), r0, r1, r2, r3);
          ptx::ldmatrix_x4_trans(vrow + (((vc + 2) ^ vsw) << 4), r4, r5, r6, r7);
          ptx::mma_16816(oa[0], a0, a1, a2, a3, r0, r1);
          ptx::mma_16816(oa[1], a0, a1, a2, a3, r2, r3);
          ptx::mma_16816(oa[2], a0, a1, a2, a3, r4, r5);
          ptx::mma_16816(oa[3], a0, a1, a2, a3, r6, r7);
        }
      }
    }
    if (tr && c0 == cbeg) p.stamps[227] = globaltimer();
    if (tr && c0 != cbeg && !more) p.stamps[235] = globaltimer();
    if (more) {
      __syncthreads();   // every warp is done with P and these value stages
      for (int j = 0; j < ATT_STAGES; ++j)
        if (!issue(c0 + ATT_STAGES + j, j, 2)) return false;
    }
  }
  // ---- normalise and store
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  __syncthreads();   // red[] still holds the last maxima
  if (qd == 0) { red[warp * 16 + g] = l_lo; red[warp * 16 + g + 8] = l_hi; }
  __syncthreads();
  float tl_lo = 0.f, tl_hi = 0.f;
#pragma unroll
  for (int w8 = 0; w8 < 8; ++w8) { tl_lo += red[w8 * 16 + g]; tl_hi += red[w8 * 16 + g + 8]; }
  if (tr) p.stamps[236] = globaltimer();
  if (kg > 0) {
    // partial result of key group kg: this thread's 16 accumulators, then (max, sum) of every row
    float* part = p.att_part + ((size_t)(kg - 1) * NROW_CTAS + unit) * ATT_PART_FLOATS;
    float4* po = reinterpret_cast<float4*>(part) + tid * 4;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) po[nt] = make_float4(oa[nt][0], oa[nt][1], oa[nt][2], oa[nt][3]);
    if (warp == 0 && qd == 0) {
      reinterpret_cast<float2*>(part + 256 * 16)[g] = make_float2(m_lo, tl_lo);
      reinterpret_cast<float2*>(part + 256 * 16)[g + 8] = make_float2(m_hi, tl_hi);
    }
    return true;
  }
  if (p.key_groups > 1) {
    // merge the other groups' partial results (they cover disjoint keys): rescale everything to the common maximum
    if (!cta_wait_event(p, issue.c, EVB(EV_PART + (unit >> 4), unit & 15), (p.key_groups - 1) * (issue.pass + 1),
                        issue.pass * NSTAGE + ST_ATT)) return false;
    if (tr) p.stamps[237] = globaltimer();
    // all loads first, then the arithmetic
    float2 ml[MAX_KEY_GROUPS - 1][2];
    float4 pv[MAX_KEY_GROUPS - 1][4];
#pragma unroll
    for (int og = 1; og < MAX_KEY_GROUPS; ++og) {
      if (og < p.key_groups) {
        const float* part = p.att_part + ((size_t)(og - 1) * NROW_CTAS + unit) * ATT_PART_FLOATS;
        ml[og - 1][0] = __ldcg(reinterpret_cast<const float2*>(part + 256 * 16) + g);
        ml[og - 1][1] = __ldcg(reinterpret_cast<const float2*>(part + 256 * 16) + g + 8);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) pv[og - 1][nt] = __ldcg(reinterpret_cast<const float4*>(part) + tid * 4 + nt);
      }
    }
#pragma unroll
    for (int og = 1; og < MAX_KEY_GROUPS; ++og) {
      if (og < p.key_groups) {
        const float2 ml_lo = ml[og - 1][0], ml_hi = ml[og - 1][1];
        const float M_lo = fmaxf(m_lo, ml_lo.x), M_hi = fmaxf(m_hi, ml_hi.x);
        const float a_lo = __expf(m_lo - M_lo), b_lo = __expf(ml_lo.x - M_lo);
        const float a_hi = __expf(m_hi - M_hi), b_hi = __expf(ml_hi.x - M_hi);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const float4 v = pv[og - 1][nt];
          oa[nt][0] = oa[nt][0] * a_lo + v.x * b_lo; oa[nt][1] = oa[nt][1] * a_lo + v.y * b_lo;
          oa[nt][2] = oa[nt][2] * a_hi + v.z * b_hi; oa[nt][3] = oa[nt][3] * a_hi + v.w * b_hi;
        }
        tl_lo = tl_lo * a_lo + ml_lo.y * b_lo; tl_hi = tl_hi * a_hi + ml_hi.y * b_hi;
        m_lo = M_lo; m_hi = M_hi;
      }
    }
  }
  if (tr) p.stamps[238] = globaltimer();
  const float il_lo = 1.0f / tl_lo, il_hi = 1.0f / tl_hi;
  __nv_bfloat16* out = o.attn + (size_t)unit * 2 * QD;   // rows m = token_local * 8 + head are contiguous
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int col = warp * 32 + nt * 8 + 2 * qd;
    *reinterpret_cast<uint32_t*>(out + (size_t)g * HD + col) = pack_bf16(oa[nt][0] * il_lo, oa[nt][1] * il_lo);
    *reinterpret_cast<uint32_t*>(out + (size_t)(g + 8) * HD + col) = pack_bf16(oa[nt][2] * il_hi, oa[nt][3] * il_hi);
  }
  ptx::fence_proxy_async_global();   // attn is read by the O projection's TMA
  return true;
}

// ------------------------------------------------------------------------------------------- GEMM CTA roles
struct Bars {
  uint32_t full, empty, tfull, tempty;   // shared-memory addresses of barrier arrays
};

__device__ __forceinline__ int stage_of(int pass, int gemm) { return pass * NSTAGE + kGemmStage[gemm]; }

struct Producer { int pass, u, b, a; uint32_t it, slot, par; bool done; };

// Tensor maps and first rows of the two 64-row halves of a unit's 128-row weight tile.
__device__ __forceinline__ void weight_rows(const Params& p, const Unit& un, int layer, const CUtensorMap*& ma,
                                            const CUtensorMap*& mb, int& ra, int& rbw) {
  if (un.gemm == G_QKV) {   // q, v: tiles of 128 consecutive output rows; k: 64 rotary dims and their partners
    if (un.tile < 16) { ma = mb = &p.maps.wq; ra = layer * QD + un.tile * 128; }
    else if (un.tile < 18) { ma = mb = &p.maps.wk; ra = layer * HD + (un.tile - 16) * 64; rbw = ra + 128; return; }  // k: dim d with d+128
    else { ma = mb = &p.maps.wv; ra = layer * HD + (un.tile - 18) * 128; }
    rbw = ra + 64;
  } else if (un.gemm == G_O) { ma = mb = &p.maps.wo; ra = layer * W + un.tile * 128; rbw = ra + 64; }
  else if (un.gemm == G_GU) { ma = &p.maps.wg; mb = &p.maps.wu; ra = rbw = layer * FF + un.tile * 64; }
  else { ma = mb = &p.maps.wd; ra = layer * W + un.tile * 128; rbw = ra + 64; }
}

// Issue weight loads in schedule order until `until` stages have been issued in total (or the schedule ends).
// A stage holds 128 weight rows x 128 k as two 64-k halves, each made of two 64-row boxes.  The thread is alone
// in its warp, so every instruction costs its full latency: everything that does not change within a unit is
// computed once per unit.
__device__ void weight_producer(const Params& p, const Ctx& c, const Unit* units, int nunits, uint32_t ring,
                                const Bars& b, Producer& st, uint32_t until, uint64_t policy, bool leader) {
  const int npass = p.n_steps * p.n_layers;
  if (nunits == 0) { st.done = true; return; }
  const bool once = PI05_NGRP(p) == 1;   // one group of observations: every weight byte is used once, mark it evict-first in L2
  while (!st.done && st.it < until) {
    if (st.pass >= PI05_CYCLES(p, npass)) { st.done = true; break; }   // st.pass counts cycles
    Unit un = units[st.u];
    int ug0, ug1;
    const int pass = st.pass - unit_groups(p, un, ug0, ug1);
    if (PI05_BATCHED && (pass < 0 || pass >= npass)) {      // the entry has no layer pass in this cycle
      if (++st.u >= nunits) { st.u = 0; ++st.pass; }
      continue;
    }
    const int stage = stage_of(pass, un.gemm);
    if (stage >= PI05_MAXSTAGE(p)) { st.done = true; break; }
    const CUtensorMap *ma, *mb;
    int ra, rbw;
    weight_rows(p, un, pass % p.n_layers, ma, mb, ra, rbw);
    int kc = (un.k0 + st.a) * KSTAGE;
    uint32_t slot = st.slot, par = st.par, it = st.it;
    int a = st.a;
    for (; a < un.nk && it < until; ++a, ++it, kc += KSTAGE) {
      if (!wait_mbar(c, b.empty + 8 * slot, par ^ 1, WAIT_W_EMPTY, stage)) { st.done = true; break; }
      const uint32_t full = b.full + 8 * slot;
      const uint32_t dst = ring + slot * V_STAGE_ALL;
      if (!leader) {
      } else if (once) {
        ptx::mbar_expect_tx(full, W_STAGE_BYTES);
        ptx::tma_load_2d_hint(dst, ma, full, kc, ra, policy);
        ptx::tma_load_2d_hint(dst + W_ATOM_BYTES / 2, mb, full, kc, rbw, policy);
        ptx::tma_load_2d_hint(dst + W_ATOM_BYTES, ma, full, kc + KATOM, ra, policy);
        ptx::tma_load_2d_hint(dst + W_ATOM_BYTES + W_ATOM_BYTES / 2, mb, full, kc + KATOM, rbw, policy);
      } else {                        // the unit's weights come again for the next observation: keep them in L2
        ptx::mbar_expect_tx(full, W_STAGE_BYTES);
        ptx::tma_load_2d(dst, ma, full, kc, ra);
        ptx::tma_load_2d(dst + W_ATOM_BYTES / 2, mb, full, kc, rbw);
        ptx::tma_load_2d(dst + W_ATOM_BYTES, ma, full, kc + KATOM, ra);
        ptx::tma_load_2d(dst + W_ATOM_BYTES + W_ATOM_BYTES / 2, mb, full, kc + KATOM, rbw);
      }
      if (++slot == V_NSTG) { slot = 0; par ^= 1; }
    }
    st.slot = slot; st.par = par; st.it = it; st.a = a;
    if (a >= un.nk) {
      st.a = 0;
      if (++st.b >= ug1 - ug0) {         // same unit again for the next group of observations, then the next unit
        st.b = 0;
        if (++st.u >= nunits) { st.u = 0; ++st.pass; }
      }
    }
  }
}

// Activation half of every stage: waits for the stage that produces the operand, then follows the same stage
// order as the weight producer.
__device__ void act_producer(const Params& p, const Ctx& c, const Unit* units, int nunits, uint32_t ring, const Bars& b,
                             bool leader) {
  const int npass = p.n_steps * p.n_layers;
  uint32_t slot = 0, par = 0;
  for (int cyc = 0; cyc < PI05_CYCLES(p, npass); ++cyc) {
    for (int u = 0; u < nunits; ++u)
    for (int gi = 0, ug0 = 0, ug1 = 1; gi < ug1 - ug0; ++gi) {   // one group of up to GN observations per round of MMAs
      Unit un = units[u];
      const int pass = cyc - unit_groups(p, un, ug0, ug1);
      if (PI05_BATCHED && (pass < 0 || pass >= npass)) break;    // the entry has no layer pass in this cycle
      const int ob0 = (ug0 + gi) * GN;
      const int stage = stage_of(pass, un.gemm);
      if (stage >= PI05_MAXSTAGE(p)) return;
      const CUtensorMap* m;
      int ev;
      unsigned target;
      if (un.gemm == G_QKV) { m = &p.maps.an_attn; ev = EV_ANA; target = NROW_CTAS * (pass + 1); }
      else if (un.gemm == G_O) { m = &p.maps.attn; ev = EV_ATT; target = NROW_CTAS * (pass + 1); }
      else if (un.gemm == G_GU) { m = &p.maps.an_ffn; ev = EV_ANF; target = NROW_CTAS * (pass + 1); }
      else { m = &p.maps.act; ev = EV_GU; target = p.n_units[G_GU] * (pass + 1); }
      const int nob = GN == 1 ? 1 : min(GN, PI05_NB(p) - ob0);
      for (int g = 0; g < nob; ++g)
        if (!wait_event(c, p.ctrl + EVB(ev, ob0 + g), target, stage)) return;
      if (ob0 == 0 && leader) trace(p, c.cta, pass, un.gemm, 0);
      ptx::fence_proxy_async_global();
      // first row of the first observation's tile: the normalised activations exist in AN_COPIES copies
      const bool copies = un.gemm == G_QKV || un.gemm == G_GU;
      const int row0 = copies ? (ob0 * AN_COPIES + c.cta % AN_COPIES) * T : ob0 * T;
      const int rstep = copies ? AN_COPIES * T : T;
      int kc = un.k0 * KSTAGE;
      for (int a = 0; a < un.nk; ++a, kc += KSTAGE) {
        if (!wait_mbar(c, b.empty + 8 * slot, par ^ 1, WAIT_A_EMPTY, stage)) return;
        const uint32_t full = b.full + 8 * slot;
        const uint32_t dst = ring + slot * V_STAGE_ALL + W_STAGE_BYTES;
        if (leader) {
          // observation g's 50 token rows land in rows 64 g .. of both 64-k atoms; the slots of observations
          // that a short last group lacks keep stale bytes, which only reach accumulator columns nobody reads
          ptx::mbar_expect_tx(full, nob * A_STAGE_TX);
#pragma unroll
          for (int g = 0; g < GN; ++g)
            if (g < nob) {
              ptx::tma_load_2d(dst + g * A_ATOM_BYTES, m, full, kc, row0 + g * rstep);
              ptx::tma_load_2d(dst + V_A_ATOM + g * A_ATOM_BYTES, m, full, kc + KATOM, row0 + g * rstep);
            }
          if (PI05_TRACE && p.stamps != nullptr && pass == 1 && c.cta == 0 && un.gemm == G_GU && a < 8) p.stamps[241 + 2 * a] = globaltimer();
        }
        if (++slot == V_NSTG) { slot = 0; par ^= 1; }
      }
      if (ob0 == 0 && leader) trace(p, c.cta, pass, un.gemm, 1);
    }
  }
}

// Returns the number of stages consumed (for the drain at exit).  One thread issues every MMA of the CTA, and a
// tcgen05 instruction costs it about 50 cycles, so the loop does one wait and one commit per eight MMAs and
// advances the shared-memory descriptors by adding constants to their low words.
__device__ uint32_t mma_issuer(const Params& p, const Ctx& c, const Unit* units, int nunits, uint32_t ring,
                               const Bars& b, uint32_t tmem, bool leader) {
  const int npass = p.n_steps * p.n_layers;
  const uint32_t idesc = ptx::umma_idesc_bf16(128, 64 * GN);
  const uint64_t adesc0 = ptx::umma_smem_desc(ring), bdesc0 = ptx::umma_smem_desc(ring + W_STAGE_BYTES);
  uint32_t it = 0, uit = 0, slot = 0, par = 0;
  for (int cyc = 0; cyc < PI05_CYCLES(p, npass); ++cyc) {
    for (int u = 0; u < nunits; ++u)
    for (int gi = 0, ug0 = 0, ug1 = 1; gi < ug1 - ug0; ++gi, ++uit) {
      Unit un = units[u];
      const int pass = cyc - unit_groups(p, un, ug0, ug1);
      if (PI05_BATCHED && (pass < 0 || pass >= npass)) break;    // the entry has no layer pass in this cycle
      const int stage = stage_of(pass, un.gemm);
      if (stage >= PI05_MAXSTAGE(p)) return it;
      const uint32_t buf = uit & 1;
      if (!wait_mbar(c, b.tempty + 8 * buf, ((uit >> 1) & 1) ^ 1, WAIT_T_EMPTY, stage)) return it;
      ptx::tc_fence_after();
      const uint32_t d = tmem + buf * (64 * GN);
      uint32_t accumulate = 0;
      for (int a = 0; a < un.nk; ++a, ++it) {
        if (!wait_mbar(c, b.full + 8 * slot, par, WAIT_W_FULL, stage)) return it;
        if (a == 0 && gi == 0 && leader) trace(p, c.cta, pass, un.gemm, 2);
        if (PI05_TRACE && leader && p.stamps != nullptr && pass == 1 && c.cta == 0 && un.gemm == G_GU && a < 8) p.stamps[240 + 2 * a] = globaltimer();
        const uint64_t ad = adesc0 + (uint64_t)(slot * (V_STAGE_ALL >> 4));
        const uint64_t bd = bdesc0 + (uint64_t)(slot * (V_STAGE_ALL >> 4));
        if (leader)
          ptx::umma_bf16_stage8<(W_ATOM_BYTES >> 4), (V_A_ATOM >> 4)>(d, ad, bd, idesc, accumulate, b.empty + 8 * slot);
        accumulate = 1u;
        if (++slot == V_NSTG) { slot = 0; par ^= 1; }
      }
      if (leader) ptx::umma_commit(b.tfull + 8 * buf);
      if (gi == 0 && leader) trace(p, c.cta, pass, un.gemm, 3);
    }
  }
  return it;
}

// Four warps (128 threads); thread r owns accumulator row r (one weight row) for all 64 token columns.
__device__ void epilogue(const Params& p, const Ctx& c, const Unit* units, int nunits, uint8_t* smem, const Bars& b,
                         uint32_t tmem) {
  const int npass = p.n_steps * p.n_layers;
  const int et = threadIdx.x - 128;          // 0..127 = accumulator row
  const int ew = et >> 5;                    // TMEM lane quadrant of this warp (warp index % 4)
  __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + OFF_STAGE);
  uint32_t uit = 0;
  for (int cyc = 0; cyc < PI05_CYCLES(p, npass); ++cyc) {
    for (int u = 0; u < nunits; ++u)
    for (int gi = 0, ug0 = 0, ug1 = 1; gi < ug1 - ug0; ++gi, ++uit) {   // one accumulator holds a group of up to GN observations
      Unit un = units[u];
      const int pass = cyc - unit_groups(p, un, ug0, ug1);
      if (PI05_BATCHED && (pass < 0 || pass >= npass)) break;    // the entry has no layer pass in this cycle
      const int ob0 = (ug0 + gi) * GN;
      const int stage = stage_of(pass, un.gemm);
      if (stage >= PI05_MAXSTAGE(p)) return;
      const uint32_t buf = uit & 1;
      const int nob = GN == 1 ? 1 : min(GN, PI05_NB(p) - ob0);
      const bool ktile = un.gemm == G_QKV && un.tile >= 16 && un.tile < 18;
      // k tiles: the RoPE table words of this thread's rotary index are fetched now, while the MMAs still run
      // (with several observations per accumulator: per observation, below)
      uint2 cs[T / 2];
      if (GN == 1 && ktile) {
        const uint2* __restrict__ rope = reinterpret_cast<const uint2*>(obs(p, ob0).rope2) + (un.tile - 16) * 64 + (et & 63);
#pragma unroll
        for (int tp = 0; tp < T / 2; ++tp) cs[tp] = __ldcg(rope + tp * (HD / 2));
      }
      const bool ok = wait_mbar(c, b.tfull + 8 * buf, (uit >> 1) & 1, WAIT_T_FULL, stage);
      {  // all 128 threads agree on whether to go on
        int any_fail;
        asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbarrier.cta.red.or.pred q, 1, 128, p;\nselp.u32 %0, 1, 0, q;\n}"
                     : "=r"(any_fail) : "r"(ok ? 0 : 1) : "memory");
        if (any_fail) return;
      }
      if (et == 0 && ob0 == 0) trace(p, c.cta, pass, un.gemm, 4);
      ptx::tc_fence_after();
#pragma unroll 1
      for (int g = 0; g < nob; ++g) {
      const int ob = ob0 + g;
      const ObsPtrs o = obs(p, ob);
      if (GN > 1 && ktile) {
        const uint2* __restrict__ rope = reinterpret_cast<const uint2*>(o.rope2) + (un.tile - 16) * 64 + (et & 63);
#pragma unroll
        for (int tp = 0; tp < T / 2; ++tp) cs[tp] = __ldcg(rope + tp * (HD / 2));
      }
      uint32_t r[64];
      {
        uint32_t lo[32], hi[32];
        const uint32_t taddr = tmem + buf * (64 * GN) + g * 64 + ((uint32_t)(ew * 32) << 16);
        ptx::tmem_ld_32x32(taddr, lo);
        ptx::tmem_ld_32x32(taddr + 32, hi);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) { r[i] = lo[i]; r[32 + i] = hi[i]; }
      }
      if (g == nob - 1) {      // the accumulator is in registers for every observation of the group
        ptx::tc_fence_before();
        ptx::mbar_arrive(b.tempty + 8 * buf);
      }
      if (et == 0 && ob == 0) trace(p, c.cta, pass, un.gemm, 5);

      if (un.gemm == G_QKV && un.tile >= 16) {
        // k / v tile over the full K: BF16 keys (with RoPE) / values straight to the buffers attention copies from
        uint32_t pk[T / 2];
#pragma unroll
        for (int i = 0; i < T / 2; ++i) pk[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        if (un.tile < 18) {
          // rows 0..63: rotary dim j = cblk*64 + row, rows 64..127: its partner j + 128; exchange through shared memory
          uint32_t* mine = reinterpret_cast<uint32_t*>(stg + et * STAGE_STRIDE);
#pragma unroll
          for (int i = 0; i < T / 2; ++i) mine[i] = pk[i];
          ptx::named_bar_sync(1, 128);
          const uint32_t* other = reinterpret_cast<const uint32_t*>(stg + (et ^ 64) * STAGE_STRIDE);
          const bool hi = et >= 64;
          const int j = (un.tile - 16) * 64 + (et & 63);
          __nv_bfloat16* dst = o.k + j + (hi ? 128 : 0);
#pragma unroll
          for (int tp = 0; tp < T / 2; ++tp) {
            // packed BF16 arithmetic on a token pair; _rn keeps every product and the sum separately rounded
            const uint32_t yw = other[tp];
            const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&pk[tp]);
            const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(&yw);
            const __nv_bfloat162 co = *reinterpret_cast<const __nv_bfloat162*>(&cs[tp].x);
            const __nv_bfloat162 si = *reinterpret_cast<const __nv_bfloat162*>(&cs[tp].y);
            const __nv_bfloat162 rot = hi ? y : __hneg2(y);                       // rotate_half: (-x2, x1)
            const __nv_bfloat162 out = __hadd2_rn(__hmul2_rn(x, co), __hmul2_rn(rot, si));
            dst[(size_t)(2 * tp) * HD] = __low2bfloat16(out);
            dst[(size_t)(2 * tp + 1) * HD] = __high2bfloat16(out);
          }
        } else {
          __nv_bfloat16* dst = o.v + (un.tile - 18) * 128 + et;
#pragma unroll
          for (int tp = 0; tp < T / 2; ++tp) {
            const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&pk[tp]);
            dst[(size_t)(2 * tp) * HD] = __low2bfloat16(x);
            dst[(size_t)(2 * tp + 1) * HD] = __high2bfloat16(x);
          }
        }
        ptx::fence_proxy_async_global();   // k and v are read by attention's bulk copies
      } else if (un.gemm != G_GU) {
        // split-K partial: FP32 reduction into an L2-resident accumulator ([T][W] for O / down, [T][2560] for QKV)
        float* acc;
        int ldacc;
        if (un.gemm == G_QKV) { acc = o.qkv_acc; ldacc = QKVW; }
        else { acc = un.gemm == G_O ? o.o_acc : o.d_acc; ldacc = W; }
        acc += un.tile * 128 + et;   // accumulator column = tile row (k tiles: 64 dims, then their 64 partners)
#pragma unroll
        for (int t = 0; t < T; ++t) ptx::red_add_f32(acc + (size_t)t * ldacc, __uint_as_float(r[t]));
      } else {
        // gate/up: rows 0..63 gate, 64..127 up of features tile*64 + (row & 63).  Exchange BF16-rounded rows through
        // shared memory (row et <-> row et ^ 64); each thread then finishes half of the tokens.
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        uint4* mine = reinterpret_cast<uint4*>(stg + et * STAGE_STRIDE);
#pragma unroll
        for (int i = 0; i < 8; ++i) mine[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        ptx::named_bar_sync(1, 128);
        const uint4* other = reinterpret_cast<const uint4*>(stg + (et ^ 64) * STAGE_STRIDE);
        uint32_t po[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) { const uint4 v = other[i]; po[4 * i] = v.x; po[4 * i + 1] = v.y; po[4 * i + 2] = v.z; po[4 * i + 3] = v.w; }
        const bool is_up = et >= 64;
        __nv_bfloat16* dst = o.act + un.tile * 64 + (et & 63);
#pragma unroll
        for (int t = 0; t < T; ++t) {
          if ((t >= 25) == is_up) {
            const float a = (t & 1) ? bf16_hi(pk[t >> 1]) : bf16_lo(pk[t >> 1]);
            const float o2 = (t & 1) ? bf16_hi(po[t >> 1]) : bf16_lo(po[t >> 1]);
            const float gv = is_up ? o2 : a, uv = is_up ? a : o2;
            dst[(size_t)t * FF] = __float2bfloat16_rn(rb(gelu_tanh(gv)) * uv);
          }
        }
        ptx::fence_proxy_async_global();   // act is read by the down projection's TMA
      }
      if (et == 0 && ob == 0) trace(p, c.cta, pass, un.gemm, 6);
      ptx::named_bar_sync(1, 128);
      if (et == 0) {
        // one signal per observation as soon as its results are stored (signalling a whole group at once was
        // measured slower: the first observation's consumers then start later)
        const int ev = un.gemm == G_QKV ? (un.tile >= 16 ? EV_KV : EV_QKV) : un.gemm == G_O ? EV_O : un.gemm == G_GU ? EV_GU : EV_DOWN;
        signal_event(p.ctrl + EVB(ev, ob));
        if (ob == 0) trace(p, c.cta, pass, un.gemm, 7);
      }
      }   // observations of the group
    }
  }
}

// ------------------------------------------------------------------------------------------- row CTA main loop
__device__ void cta_signal(const Params& p, int ev, int b) {
  __syncthreads();
  if (threadIdx.x == 0 && ev != PI05_DROP(p)) signal_event(p.ctrl + EVB(ev, b));
}

// One layer-pass step of a row CTA for one observation.  Each returns false when a wait gave up.
__device__ __forceinline__ bool row_attention(const Params& p, const Ctx& c, uint8_t* smem, int unit, int pass, int ob,
                                              int kg, AttBars& bars, bool stamp0) {
  const int layer = pass % p.n_layers, npc = (p.prefix + 63) / 64, sbase = 6 + pass * NSTAGE;
  const ObsPtrs o = obs(p, ob);
  const bool stamp = stamp0 && ob == 0;
  // chunks 0..npc-1 are prefix keys, chunk npc the suffix keys.  With key groups the chunks are cut into contiguous
  // shares; group 0, which merges and goes on with the residual, takes the last one (it contains the suffix chunk,
  // the one that arrives last), group g >= 1 takes share g - 1.
  const int KG = p.key_groups, total = npc + 1, share = kg == 0 ? KG - 1 : kg - 1;
  const int cbeg = total * share / KG, cend = total * (share + 1) / KG;
  AttChunkIssue issue{p, o, c, smem, bars, layer, npc, pass, cend};
  // prefix chunks do not depend on this layer's QKV: fetch them before waiting
  const int nearly = max(0, min(min(cend, npc) - cbeg, ATT_STAGES));
  for (int j = 0; j < nearly; ++j) issue(cbeg + j, j);
  if (!cta_wait_event(p, c, EVB(EV_QKV, ob), (p.n_units[G_QKV] - NKVTILES) * (pass + 1), pass * NSTAGE + ST_ATT)) {
    att_drain(c, smem, bars, pass * NSTAGE + ST_ATT);
    return false;
  }
  if (stamp && sbase + ST_QKV < 64) p.stamps[sbase + ST_QKV] = globaltimer();
  build_q(o, smem, unit);                               // q straight from the FP32 sums
  const bool tr = stamp && pass == 1;
  if (!attention_unit(p, o, smem, unit, issue, cbeg, nearly, kg, tr)) {
    att_drain(c, smem, bars, pass * NSTAGE + ST_ATT);
    return false;
  }
  if (tr) p.stamps[228] = globaltimer();
  if (kg > 0) {
    __syncthreads();
    if (threadIdx.x == 0) signal_event(p.ctrl + EVB(EV_PART + (unit >> 4), unit & 15));
  } else {
    cta_signal(p, EV_ATT, ob);
  }
  if (tr) p.stamps[229] = globaltimer();
  if (stamp && sbase + ST_ATT < 64) p.stamps[sbase + ST_ATT] = globaltimer();
  return true;
}

__device__ __forceinline__ bool row_residual(const Params& p, const Ctx& c, uint8_t* smem, int unit, int pass, int ob,
                                             int mode, float (&hn)[8], bool stamp0) {
  const int layer = pass % p.n_layers, step = pass / p.n_layers, sbase = 6 + pass * NSTAGE;
  const ObsPtrs o = obs(p, ob);
  const bool stamp = stamp0 && ob == 0;
  const bool first = mode == ROW_ATT;
  RowMod rm;
  row_prefetch(p, mode, step, layer, rm);
  if (!cta_wait_event(p, c, EVB(first ? EV_O : EV_DOWN, ob), p.n_units[first ? G_O : G_DOWN] * (pass + 1),
                      pass * NSTAGE + (first ? ST_RATT : ST_RFFN))) return false;
  if (stamp && sbase + (first ? ST_O : ST_DOWN) < 64) p.stamps[sbase + (first ? ST_O : ST_DOWN)] = globaltimer();
  if (!row_op(p, c, o, smem, unit, mode, step, layer, pass, hn, rm)) return false;
  if (stamp && pass == 1 && first) p.stamps[231] = globaltimer();
  ptx::fence_proxy_async_global();
  cta_signal(p, first ? EV_ANF : EV_ANA, ob);
  if (stamp && pass == 1 && first) p.stamps[232] = globaltimer();
  if (stamp && sbase + (first ? ST_RATT : ST_RFFN) < 64) p.stamps[sbase + (first ? ST_RATT : ST_RFFN)] = globaltimer();
  return true;
}

// Row CTA `unit` of group `group`: attention and the two residual operations of every layer pass for the
// observations group, group + row_groups, ...  With several observations the residual after the O projection of
// one observation is done right after the attention of the next one, so that the gate/up GEMM of the first can
// start while the others are still in attention.  (The GEMM CTAs run a pass as q(all observations), O(all),
// gate/up(all), down(all); every wait below is for something earlier in that order than anything still queued.)
__device__ void row_cta(const Params& p, const Ctx& c, uint8_t* smem, int unit, int group, float (&hn)[8]) {
  const int npass = p.n_steps * p.n_layers, G = PI05_NG(p);
  AttBars bars;
  for (int i = threadIdx.x; i < PI05_NB(p) * p.pages_per_obs; i += THREADS)   // the page table, kept in shared memory
    reinterpret_cast<int*>(smem + OFF_PAGETAB)[i] = p.page_table[i];
  if (threadIdx.x == 0) {
    for (int j = 0; j < 2 * ATT_STAGES; ++j) ptx::mbar_init(ptx::smem_u32(smem + OFF_ATTBARS) + 8 * j, 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (p.key_groups > 1 && group > 0) {
    // one observation, long prefix: this group only contributes its share of the keys to every attention
    for (int pass = 0; pass < npass; ++pass) {
      if (pass * NSTAGE + ST_ATT >= PI05_MAXSTAGE(p)) return;
      if (!row_attention(p, c, smem, unit, pass, 0, group, bars, false)) return;
    }
    return;
  }
  const bool stamp0 = PI05_TRACE && p.stamps != nullptr && unit == 0 && group == 0 && threadIdx.x == 0;
  const int nobs = (PI05_NB(p) - group + G - 1) / G;       // observations of this group
  if (PI05_BATCHED && p.stream_split > 0) {
    // Two-stream schedule.  The GEMM CTAs run, cycle after cycle, q(A) gate/up(B, pass before) O(A) down(B, pass before)
    // gate/up(A) q(B) down(A) O(B): between a phase and the one that depends on it through row CTAs there is always a
    // phase of the other stream.  The row CTAs follow in the order in which those phases feed them.
    // op: 0 attention(A) 1 first residual(A) 2 second residual(B, pass before) 3 attention(B) 4 second residual(A)
    //     5 first residual(B)
    for (int cyc = 0; cyc <= npass; ++cyc)
      for (int op = 0; op < 6; ++op) {
        const int stream = (0x2c >> op) & 1;                        // ops 2, 3, 5 serve stream B
        const int pass = op == 2 ? cyc - 1 : cyc;
        if (pass < 0 || pass >= npass) continue;
        for (int k = 0; k < nobs; ++k) {
          const int ob = group + k * G;
          if (((ob / GN < p.stream_split) ? 0 : 1) != stream) continue;
          if (op == 0 || op == 3) { if (!row_attention(p, c, smem, unit, pass, ob, 0, bars, false)) return; }
          else if (!row_residual(p, c, smem, unit, pass, ob, (op == 1 || op == 5) ? ROW_ATT : ROW_FFN, hn, false)) return;
        }
      }
    return;
  }
  for (int pass = 0; pass < npass; ++pass) {
    if (pass * NSTAGE + ST_ATT >= PI05_MAXSTAGE(p)) return;
    const bool do_ratt = pass * NSTAGE + ST_RATT < PI05_MAXSTAGE(p);
    if (PI05_BATCHED && p.row_order == 1) {
      for (int k = 0; k < nobs; ++k)
        if (!row_attention(p, c, smem, unit, pass, group + k * G, 0, bars, stamp0)) return;
      for (int k = 0; k < nobs && do_ratt; ++k)
        if (!row_residual(p, c, smem, unit, pass, group + k * G, ROW_ATT, hn, stamp0)) return;
    } else
    for (int k = 0; k <= nobs; ++k) {                   // attention of observation k, residual of observation k - 1
      if (k < nobs && !row_attention(p, c, smem, unit, pass, group + k * G, 0, bars, stamp0)) return;
      if (k >= 1 && do_ratt && !row_residual(p, c, smem, unit, pass, group + (k - 1) * G, ROW_ATT, hn, stamp0)) return;
    }
    if (pass * NSTAGE + ST_RFFN >= PI05_MAXSTAGE(p)) return;
    for (int k = 0; k < nobs; ++k)
      if (!row_residual(p, c, smem, unit, pass, group + k * G, ROW_FFN, hn, stamp0)) return;
  }
}

// ------------------------------------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(THREADS, 1) pi05_chunk_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int ncta = gridDim.x;
  // which CTA of the schedule this block plays: by default its own index; permuted, the two blocks of a cluster
  // (a TPC) are CTA i and CTA grid / 2 + i, e.g. a gate/up CTA next to a light one
  const int cta = p.cta_perm ? (int)(blockIdx.x >> 1) + (int)(blockIdx.x & 1) * (ncta >> 1) : (int)blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_gemm = cta < p.n_gemm_ctas;
  const Ctx c{p.ctrl, p.wait_limit, cta, (unsigned)p.poll_ns};
  const bool stamp = PI05_TRACE && p.stamps != nullptr && cta == p.n_gemm_ctas && tid == 0;
  if (stamp) p.stamps[0] = globaltimer();

  __shared__ uint32_t s_tmem;
  __shared__ uint32_t s_issued, s_consumed;
  Bars b;
  {
    const uint32_t base = ptx::smem_u32(smem + OFF_BARS);
    b.full = base; b.empty = base + 8 * NSTG; b.tfull = base + 16 * NSTG; b.tempty = b.tfull + 16;
  }
  const uint32_t ring = ptx::smem_u32(smem + OFF_RING);
  const Unit* units = p.sched + (size_t)cta * MAX_UNITS;
  const int nunits = is_gemm ? p.sched_n[cta] : 0;

  if (tid == 0) {
    s_issued = 0; s_consumed = 0;
    for (int i = 0; i < V_NSTG; ++i) { ptx::mbar_init(b.full + 8 * i, 2); ptx::mbar_init(b.empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { ptx::mbar_init(b.tfull + 8 * i, 1); ptx::mbar_init(b.tempty + 8 * i, 128); }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_shared();
  }
  if (is_gemm && warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&s_tmem), V_TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = s_tmem;

  // The first ring of weights does not depend on anything: start streaming before the prologue.
  Producer prod{0, 0, 0, 0, 0u, 0u, 0u, false};
  uint64_t policy = 0;
  const bool leader = ptx::elect_one();     // every warp is converged here
  if (is_gemm && warp == 0) {
    policy = ptx::policy_evict_first();
    weight_producer(p, c, units, nunits, ring, b, prod, V_NSTG, policy, leader);
  }

  // ---------------- prologue: tables, time MLP, all modulation rows (FP32 weights streamed once)
  bool ok = true;
  prologue_tables(p, cta, ncta);
  ok = grid_event(p, c, EV_P0, ncta);
  if (stamp) p.stamps[1] = globaltimer();
  if (ok) { matvec10<0>(p, p.temb, smem, cta, ncta); ok = grid_event(p, c, EV_P1, ncta); }
  if (stamp) p.stamps[2] = globaltimer();
  if (ok) { matvec10<1>(p, p.hid, smem, cta, ncta); ok = grid_event(p, c, EV_P2, ncta); }
  if (stamp) p.stamps[3] = globaltimer();
  if (ok) { matvec10<2>(p, p.cond, smem, cta, ncta); ok = grid_event(p, c, EV_P3, ncta); }
  if (stamp) p.stamps[4] = globaltimer();

  if (ok) {
    if (is_gemm) {
      // Warps 0-2 run their loops as whole (converged) warps and one elected lane issues the TMA / tcgen05
      // instructions: with warp-uniform control flow the compiler keeps descriptors and coordinates in uniform
      // registers, which those instructions read; the same loops run by a single lane issued ~35 % slower.
      if (warp == 0) {
        weight_producer(p, c, units, nunits, ring, b, prod, 0xffffffffu, policy, leader);
        if (leader) s_issued = prod.it;
      } else if (warp == 1) {
        const uint32_t consumed = mma_issuer(p, c, units, nunits, ring, b, tmem, leader);
        if (leader) s_consumed = consumed;
      } else if (warp == 2) {
        act_producer(p, c, units, nunits, ring, b, leader);
      } else if (warp >= 4) {
        epilogue(p, c, units, nunits, smem, b, tmem);
      }
    } else {
      const int unit = (cta - p.n_gemm_ctas) % NROW_CTAS, group = (cta - p.n_gemm_ctas) / NROW_CTAS;
      float hn[8];
      RowMod none;
      for (int ob = group; ob < PI05_NB(p); ob += PI05_NG(p)) {
        row_op(p, c, obs(p, ob), smem, unit, ROW_INIT, 0, 0, 0, hn, none);
        ptx::fence_proxy_async_global();
        cta_signal(p, EV_ANA, ob);
      }
      if (stamp) p.stamps[5] = globaltimer();
      row_cta(p, c, smem, unit, group, hn);
    }
  } else if (is_gemm && warp == 0 && leader) {
    s_issued = prod.it;
  }

  // ---------------- teardown: drain loads still in flight, free TMEM, last CTA out clears the counters
  __syncthreads();
  if (is_gemm && warp == 0 && lane == 0 && s_issued != s_consumed) {
    // Only after an aborted run: weight loads were issued whose stage was never consumed.  A stage's barrier completes
    // when both halves have arrived and every byte has landed; the activation half may never come, so arrive in its
    // place and wait (bounded) for the weights.  If the activation half did come, the barrier has completed already
    // and the extra arrival falls into a phase nobody will use.
    for (uint32_t it = s_consumed; it != s_issued; ++it) {
      const uint32_t s = it % (uint32_t)V_NSTG;
      ptx::mbar_arrive(b.full + 8 * s);
      drain_mbar(b.full + 8 * s, (it / (uint32_t)V_NSTG) & 1u, p.wait_limit);
    }
  }
  __syncthreads();
  if (is_gemm && warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, V_TMEM_COLS);
  }
  if (tid == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(p.ctrl + EVW(EV_EXIT), 1u);
    if (prev == (unsigned)ncta - 1) {
      __threadfence();
      if (ptx::ld_relaxed(p.ctrl) != 0u) {
        // a bounded wait gave up somewhere: whoever reads the output must not mistake an earlier chunk's actions for
        // this one's
        for (int i = 0; i < PI05_NB(p) * T * ADIM; ++i) p.ob.actions[i] = __int_as_float(0x7fc00000);
      }
      for (int e = 0; e < NEVENTS * MAXB; ++e) p.ctrl[32 * (1 + e)] = 0u;
      __threadfence();
    }
  }
}

#undef PI05_NB
#undef PI05_NGRP
#undef PI05_CYCLES
#undef PI05_NG
#undef PI05_MAXSTAGE
#undef PI05_DROP
