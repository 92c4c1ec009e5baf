// Gemma-2B prefix-LM prefill on B200 (sm_100a): the step before the action chunk, which turns the embedded prefix
// (image tokens + prompt) into the per-layer key / value cache the chunk engine attends over.
//
// Semantics follow the reference's eager definition (reference/pi05.py:167-195): per layer RMSNorm, q / k / v projections,
// RoPE at the positions of the valid tokens, bidirectional attention among valid tokens, O projection + residual, and
// (except after the last layer) the GeGLU MLP + residual; every matmul output, product and sum is rounded to BF16 where
// the reference's BF16 tensors round.  The outputs are the post-RoPE keys and the values, [layers, tokens, 1, 256] BF16,
// the layout pi05_bind takes as inputs 22 and 23, so the chunk engine chains after this without a copy.
//
// Structure (all new; the reference runs this part in eager PyTorch):
//   * one tcgen05 GEMM kernel, persistent over output tiles of 128 tokens x 256 (or 128) features: warp 0 streams both
//     operands with TMA through a 4- or 6-stage shared-memory ring, warp 1 issues M128 x N256 (N128) x K16 MMAs into one
//     of two TMEM accumulators, four epilogue warps read the other one; the epilogues fuse what follows the matmul -
//     RoPE and the scatter into q / k / v, GeGLU, or the residual add; it also runs as a stream-K launch (a tile's k
//     blocks spread over several CTAs) and, for the three big GEMMs, on CTA pairs (cta_group::2: 256-token tiles, each
//     CTA loading half of the weight rows);
//   * a row kernel for the Gemma RMSNorm, a table kernel for the RoPE factors;
//   * an attention kernel of 128 query rows (16 tokens x 8 heads over the one KV head) per CTA: tcgen05 MMAs for Q K^T and
//     P V over 64-key chunks staged by TMA, two passes over the keys (row maxima, then probabilities), one thread per row.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <new>
#include <string>
#include <utility>

#include "../../include/pi05_b200.h"
#include "ptx_sm100.cuh"

#include "pi05_common.cuh"
using namespace pi05;

#ifndef PI05_PREFILL_OVERLAP
#define PI05_PREFILL_OVERLAP 1     // 0: every kernel waits for the one before it to finish before it starts (for A/B runs)
#endif

namespace pf {

constexpr int H = 2048;            // Gemma-2B width
constexpr int FFN = 16384;         // MLP width
constexpr int LAYERS = 18;
constexpr int BM = 128;            // tokens per output tile (MMA M)
constexpr int BK = 64;             // k per pipeline stage (one 128-byte swizzle row)
constexpr int GEMM_THREADS = 192;  // warp 0 producer, warp 1 MMA issuer, warps 2..5 epilogue
constexpr int RING_BYTES = 192 * 1024;

enum { EPI_QKV = 0, EPI_RESID = 1, EPI_GEGLU = 2 };

struct GemmParams {
  CUtensorMap a;                   // activations [tokens, K] BF16, box {64, 128}
  CUtensorMap b0, b1;              // weights [rows, K] BF16, box {64, BN / 2}: the two halves of a tile's BN rows
  CUtensorMap b2, b3;              // EPI_QKV: wk, wv (b0 = b1 = wq)
  int tokens, kblocks, n_tiles, m_tiles, layer;
  // epilogue operands
  __nv_bfloat16* x;                // EPI_RESID: residual stream [tokens, H], updated in place
  __nv_bfloat16* act;              // EPI_GEGLU: [tokens, FFN]
  __nv_bfloat16 *q, *k, *v;        // EPI_QKV: q [tokens, 2048]; k, v: this layer's [tokens, 256]
  __nv_bfloat16* vt;               // EPI_QKV: the layer's values once more as V^T [256, vt_stride] for the attention's MMAs
  int vt_stride;
  const uint32_t* rope;            // [tokens][128]: cos BF16 | sin BF16 << 16
  unsigned int* status;
  long long wait_limit;
  // stream-K launches: partial sums [CTA][128 x BN] FP32 and one flag per CTA, which holds the number of the launch (of
  // this prefill) whose partial sums the CTA wrote last
  float* sk_partial;
  unsigned int* sk_flags;
  unsigned int sk_epoch;
};

__device__ __forceinline__ float rb(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float lo16(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi16(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float gelu_tanh(float x) {
  const float z = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(z));
}

// Bounded wait on an mbarrier of this CTA; a wait that runs out records (kind, where) once and every later wait returns.
__device__ __forceinline__ bool wait_bar(unsigned int* status, long long limit, uint32_t bar, uint32_t parity, int kind) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (unsigned i = 0;; ++i) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (ptx::ld_relaxed(status) != 0u) return false;
      if (clock64() - t0 > limit) {
        if (atomicCAS(status, 0u, (unsigned)kind) == 0u) status[1] = blockIdx.x;
        return false;
      }
    }
  }
}

// Four K = 16 MMAs over one 64-k stage (32-byte steps inside the 128-byte swizzle row) and the commit that frees it.
__device__ __forceinline__ void umma_stage4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate, uint32_t commit_bar) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "add.u64 a1, %1, 2;\n add.u64 a2, %1, 4;\n add.u64 a3, %1, 6;\n"
      "add.u64 b1, %2, 2;\n add.u64 b2, %2, 4;\n add.u64 b3, %2, 6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, 1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, 1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, 1;\n"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(commit_bar) : "memory");
}

// The fused epilogue of one output tile: this thread's token row of the FP32 accumulator (TMEM lanes of its warp, BN
// columns from t0) becomes the layer's next tensor.  `nt` is the tile's index along the features.
template <int EPI, int BN>
__device__ __forceinline__ void epilogue_row(const GemmParams& p, uint32_t t0, int nt, int token, bool live) {
  if (EPI == EPI_RESID) {
    // x += bf16(acc), rounded as the reference's BF16 add does; the old values of the next 32 columns are requested
    // before this chunk's are used (a thread's row is 4 KB away from its neighbour's, so these loads are slow ones)
    __nv_bfloat16* xr = p.x + (size_t)(live ? token : 0) * H + nt * BN;
    uint4 old[4], nxt[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) old[j] = reinterpret_cast<const uint4*>(xr)[j];
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      const int cn = c + 32 < BN ? c + 32 : c;
#pragma unroll
      for (int j = 0; j < 4; ++j) nxt[j] = reinterpret_cast<const uint4*>(xr + cn)[j];
      uint32_t r[32];
      ptx::tmem_ld_32x32(t0 + c, r);
      ptx::tmem_wait_ld();
      if (live) {
        uint4* dst = reinterpret_cast<uint4*>(xr + c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t ow[4] = {old[j].x, old[j].y, old[j].z, old[j].w};
          uint32_t nw[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a = rb(lo16(ow[e]) + rb(__uint_as_float(r[8 * j + 2 * e])));
            const float b = rb(hi16(ow[e]) + rb(__uint_as_float(r[8 * j + 2 * e + 1])));
            nw[e] = pack2(a, b);
          }
          dst[j] = make_uint4(nw[0], nw[1], nw[2], nw[3]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) old[j] = nxt[j];
    }
  } else {
    // QKV and GeGLU need columns c and c + BN / 2 of the tile together (rotary partner, gate with up)
    const bool vhead = EPI == EPI_QKV && nt >= 9;
#pragma unroll 1
    for (int c = 0; c < BN / 2; c += 32) {
      uint32_t r1[32], r2[32];
      ptx::tmem_ld_32x32(t0 + c, r1);
      ptx::tmem_ld_32x32(t0 + BN / 2 + c, r2);
      ptx::tmem_wait_ld();
      if (!live) continue;
      uint32_t o1[16], o2[16];
      if (EPI == EPI_GEGLU) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float g0 = rb(__uint_as_float(r1[2 * j])), g1 = rb(__uint_as_float(r1[2 * j + 1]));
          const float u0 = rb(__uint_as_float(r2[2 * j])), u1 = rb(__uint_as_float(r2[2 * j + 1]));
          o1[j] = pack2(rb(gelu_tanh(g0)) * u0, rb(gelu_tanh(g1)) * u1);
        }
        uint4* dst = reinterpret_cast<uint4*>(p.act + (size_t)token * FFN + nt * (BN / 2) + c);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o1[4 * j], o1[4 * j + 1], o1[4 * j + 2], o1[4 * j + 3]);
      } else {
        if (vhead) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            o1[j] = pack2(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
            o2[j] = pack2(__uint_as_float(r2[2 * j]), __uint_as_float(r2[2 * j + 1]));
          }
          // V^T: a warp's 32 tokens are neighbours in every dim row
          unsigned short* t1 = reinterpret_cast<unsigned short*>(p.vt) + (size_t)c * p.vt_stride + token;
          unsigned short* t2 = t1 + (size_t)128 * p.vt_stride;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            t1[(size_t)(2 * j) * p.vt_stride] = (unsigned short)(o1[j] & 0xffffu);
            t1[(size_t)(2 * j + 1) * p.vt_stride] = (unsigned short)(o1[j] >> 16);
            t2[(size_t)(2 * j) * p.vt_stride] = (unsigned short)(o2[j] & 0xffffu);
            t2[(size_t)(2 * j + 1) * p.vt_stride] = (unsigned short)(o2[j] >> 16);
          }
        } else {
          // RoPE (reference/pi05.py:218-229 on BF16 tensors): x cos + rotate_half(x) sin, every product and the
          // sum rounded to BF16; dims c.. pair with dims 128 + c..
          const uint4* cs4 = reinterpret_cast<const uint4*>(p.rope + (size_t)token * 128 + c);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const uint4 w4 = __ldg(cs4 + j4);
            const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              float a[2], b[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const uint32_t w = ws[2 * h + e];
                const float co = lo16(w), si = hi16(w);
                const float x1 = rb(__uint_as_float(r1[4 * j4 + 2 * h + e])), x2 = rb(__uint_as_float(r2[4 * j4 + 2 * h + e]));
                a[e] = rb(rb(x1 * co) + rb(-x2 * si));
                b[e] = rb(rb(x2 * co) + rb(x1 * si));
              }
              o1[2 * j4 + h] = pack2(a[0], a[1]);
              o2[2 * j4 + h] = pack2(b[0], b[1]);
            }
          }
        }
        __nv_bfloat16* base = nt < 8 ? p.q + (size_t)token * 2048 + nt * 256
                                     : (nt == 8 ? p.k : p.v) + (size_t)token * 256;
        uint4* d1 = reinterpret_cast<uint4*>(base + c);
        uint4* d2 = reinterpret_cast<uint4*>(base + 128 + c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          d1[j] = make_uint4(o1[4 * j], o1[4 * j + 1], o1[4 * j + 2], o1[4 * j + 3]);
          d2[j] = make_uint4(o2[4 * j], o2[4 * j + 1], o2[4 * j + 2], o2[4 * j + 3]);
        }
      }
    }
  }
}

// The work of one CTA of a GEMM launch, as segments (tile, first k block, one past the last k block).
// SK = false: whole tiles blockIdx.x, blockIdx.x + gridDim.x, ...  SK = true ("stream-K"): the launch's tiles x k blocks,
// taken as one sequence of units, are cut into gridDim.x contiguous, equal ranges, so that a GEMM with fewer tiles than
// the GPU has SMs (or a ragged last wave) still keeps every SM busy for the same time.  A range that begins inside a
// tile makes its CTA a contributor to that tile: it leaves its FP32 partial sums in the workspace and raises a flag.  A
// range that ends inside a tile (having begun it) makes its CTA the tile's owner: it adds the partial sums of the
// CTAs that follow it, whose ranges hold the rest of the tile, and runs the fused epilogue.  An owner's wait is for CTAs
// of higher index only, and the partial segment those wait for nobody, so no wait can close a circle.
template <bool SK>
struct Segments {
  int kblocks, ntiles, tile, stride;
  long long u, uend;
  __host__ __device__ Segments(int kblocks_, int ntiles_, int cta, int ctas) : kblocks(kblocks_), ntiles(ntiles_) {
    tile = cta; stride = ctas; u = uend = 0;
    if (SK) {
      const long long total = (long long)ntiles * kblocks;
      u = total * cta / ctas;
      uend = total * (cta + 1) / ctas;
    }
  }
  __host__ __device__ bool next(int& t, int& kb0, int& kb1) {
    if (SK) {
      if (u >= uend) return false;
      t = (int)(u / kblocks);
      kb0 = (int)(u - (long long)t * kblocks);
      const long long rest = uend - u;
      kb1 = rest < kblocks - kb0 ? kb0 + (int)rest : kblocks;
      u += kb1 - kb0;
      return true;
    }
    if (tile >= ntiles) return false;
    t = tile; kb0 = 0; kb1 = kblocks; tile += stride;
    return true;
  }
};

// out[tokens, N] = A[tokens, K] . W[N, K]^T with a fused epilogue; tile = 128 tokens x BN features.
template <int EPI, int BN, bool SK>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
  constexpr int NST = RING_BYTES / STAGE;
  constexpr int TCOLS = 2 * BN;
  static_assert(NST >= 4 && TCOLS <= 512, "ring / TMEM capacity");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bars[2 * NST + 6];
  __shared__ uint32_t s_tmem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ring = ptx::smem_u32(smem);
  const uint32_t full = ptx::smem_u32(bars), empty = full + 8 * NST, tfull = empty + 8 * NST, tempty = tfull + 16;
  const uint32_t fix = tempty + 16;      // stream-K: a peer's partial sums have landed in half of the ring
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) { ptx::mbar_init(full + 8 * i, 1); ptx::mbar_init(empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(tfull + 8 * i, 1); ptx::mbar_init(tempty + 8 * i, 128); ptx::mbar_init(fix + 8 * i, 1);
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_shared();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&s_tmem), TCOLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = s_tmem;
  const int ntiles = p.n_tiles * p.m_tiles;
  const bool leader = ptx::elect_one();
  // everything up to here overlapped the tail of the kernel before; its outputs are read from here on
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();
  Segments<SK> segs(p.kblocks, ntiles, (int)blockIdx.x, (int)gridDim.x);
  int tile, kb0, kb1;

  if (warp == 0) {
    // ---- producer: both operands of every stage, segment after segment (consecutive tiles share the weight rows)
    uint32_t slot = 0, par = 0;
    while (segs.next(tile, kb0, kb1)) {
      const int nt = tile / p.m_tiles, mt = tile % p.m_tiles;
      const CUtensorMap *m0 = &p.b0, *m1 = &p.b1;
      int r0, r1;
      if (EPI == EPI_QKV) {            // tile = one head of 256 features: q heads 0..7 (wq), then k (wk), then v (wv)
        if (nt >= 9) { m0 = m1 = &p.b3; r0 = p.layer * 256; }
        else if (nt == 8) { m0 = m1 = &p.b2; r0 = p.layer * 256; }
        else r0 = p.layer * 2048 + nt * 256;
        r1 = r0 + 128;
      } else if (EPI == EPI_GEGLU) {   // 128 gate rows and the matching 128 up rows
        r0 = r1 = p.layer * FFN + nt * (BN / 2);
      } else {
        r0 = p.layer * H + nt * BN;
        r1 = r0 + BN / 2;
      }
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!wait_bar(p.status, p.wait_limit, empty + 8 * slot, par ^ 1, 1)) return;
        if (leader) {
          const uint32_t bar = full + 8 * slot, dst = ring + slot * STAGE;
          ptx::mbar_expect_tx(bar, STAGE);
          ptx::tma_load_2d(dst, &p.a, bar, kb * BK, mt * BM);
          ptx::tma_load_2d(dst + A_BYTES, m0, bar, kb * BK, r0);
          ptx::tma_load_2d(dst + A_BYTES + B_BYTES / 2, m1, bar, kb * BK, r1);
        }
        if (++slot == NST) { slot = 0; par ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    const uint32_t idesc = ptx::umma_idesc_bf16(BM, BN);
    const uint64_t adesc0 = ptx::umma_smem_desc(ring), bdesc0 = ptx::umma_smem_desc(ring + A_BYTES);
    uint32_t slot = 0, par = 0, it = 0;
    bool ok = true;
    while (ok && segs.next(tile, kb0, kb1)) {
      const uint32_t buf = it & 1;
      if (!wait_bar(p.status, p.wait_limit, tempty + 8 * buf, ((it >> 1) & 1) ^ 1, 2)) break;
      ptx::tc_fence_after();
      const uint32_t d = tmem + buf * BN;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!wait_bar(p.status, p.wait_limit, full + 8 * slot, par, 3)) { ok = false; break; }
        const uint64_t off = (uint64_t)(slot * (STAGE >> 4));
        if (leader) umma_stage4(d, adesc0 + off, bdesc0 + off, idesc, kb > kb0 ? 1u : 0u, empty + 8 * slot);
        if (++slot == NST) { slot = 0; par ^= 1; }
      }
      if (ok && leader) ptx::umma_commit(tfull + 8 * buf);
      ++it;
    }
  } else {
    // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) ..; thread = token row of the tile
    const int quad = warp & 3, row = quad * 32 + lane;
    uint32_t it = 0;
    while (segs.next(tile, kb0, kb1)) {
      const int nt = tile / p.m_tiles, mt = tile % p.m_tiles;
      const uint32_t buf = it & 1;
      const int token = mt * BM + row;
      const bool live = token < p.tokens;
      if (!wait_bar(p.status, p.wait_limit, tfull + 8 * buf, (it >> 1) & 1, 4)) break;
      ++it;
      ptx::tc_fence_after();
      const uint32_t t0 = tmem + buf * BN + ((uint32_t)(quad * 32) << 16);
      // partial sums of a tile in the workspace: [CTA][column][row] FP32, so that a warp's 32 rows of one column are one line
      if (SK && kb0 > 0) {
        // contributor: the tile's owner is a CTA before this one
        float* mine = p.sk_partial + (size_t)blockIdx.x * (BM * BN) + row;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(t0 + c, r);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(mine + (size_t)(c + j) * BM, __uint_as_float(r[j]));
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(tempty + 8 * buf);
        ptx::named_bar_sync(1, 128);                       // every row's partial sums are written ...
        if (tid == 64) ptx::st_release(p.sk_flags + blockIdx.x, p.sk_epoch);   // ... before the flag says so
        continue;
      }
      if (SK && kb1 < p.kblocks) {
        // owner of a tile whose later k blocks went to the CTAs after this one (their ranges begin inside this tile):
        // wait for their flags (bounded), then pull their partial sums through the ring - which is idle, this being the
        // CTA's last segment with all its MMAs complete - half a tile at a time, and add them to the accumulator in TMEM
        const long long total = (long long)ntiles * p.kblocks, tile_end = (long long)(tile + 1) * p.kblocks;
        const int first_peer = blockIdx.x + 1;
        int npeers = 0;
        while (first_peer + npeers < (int)gridDim.x && total * (first_peer + npeers) / gridDim.x < tile_end) ++npeers;
        bool ok = true;
        for (int j = 0; ok && j < npeers; ++j) {
          const long long t_start = clock64();
          while (ptx::ld_acquire(p.sk_flags + first_peer + j) != p.sk_epoch) {
            if (ptx::ld_relaxed(p.status) != 0u) { ok = false; break; }
            if (clock64() - t_start > p.wait_limit) {
              if (atomicCAS(p.status, 0u, 12u) == 0u) p.status[1] = blockIdx.x;
              ok = false;
              break;
            }
            __nanosleep(20);
          }
        }
        if (!ok) break;
        constexpr int HALF_COLS = BN / 2, HALF_BYTES = HALF_COLS * BM * 4;
        static_assert(2 * HALF_BYTES <= RING_BYTES, "two half tiles of partial sums fit the ring");
        const int items = 2 * npeers;
        auto fetch = [&](int k) {   // item k = (peer k / 2, half k % 2) into ring half k % 2
          const float* src = p.sk_partial + (size_t)(first_peer + (k >> 1)) * (BM * BN) + (size_t)(k & 1) * HALF_COLS * BM;
          const uint32_t bar = fix + 8 * (k & 1), dst = ring + (k & 1) * HALF_BYTES;
          ptx::mbar_expect_tx(bar, HALF_BYTES);
          for (int q4 = 0; q4 < HALF_BYTES; q4 += 16384) ptx::bulk_load(dst + q4, reinterpret_cast<const uint8_t*>(src) + q4, 16384, bar);
        };
        if (tid == 64) { fetch(0); if (items > 1) fetch(1); }
        for (int k = 0; ok && k < items; ++k) {
          if (!wait_bar(p.status, p.wait_limit, fix + 8 * (k & 1), (k >> 1) & 1, 13)) { ok = false; break; }
          const float* part = reinterpret_cast<const float*>(smem + (k & 1) * HALF_BYTES) + row;
#pragma unroll 1
          for (int c = 0; c < HALF_COLS; c += 32) {
            uint32_t r[32];
            const uint32_t ta = t0 + (k & 1) * HALF_COLS + c;
            ptx::tmem_ld_32x32(ta, r);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + part[(c + j) * BM]);
            ptx::tmem_st_32x32(ta, r);
          }
          ptx::tmem_wait_st();                             // the next peer's pass reads these columns again
          ptx::named_bar_sync(1, 128);                     // everybody has read this half of the ring
          if (tid == 64 && k + 2 < items) fetch(k + 2);
        }
        if (!ok) break;
      }
      epilogue_row<EPI, BN>(p, t0, nt, token, live);
      ptx::tc_fence_before();
      ptx::mbar_arrive(tempty + 8 * buf);
    }
  }
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, TCOLS);
  }
}

// The same GEMM on CTA pairs (cta_group::2): a tile is 256 tokens x BN features, each CTA of the pair owning 128 of the
// tokens and loading, besides its rows of A, only HALF of the tile's weight rows - the MMA reads the other half from the
// partner's shared memory.  A CTA's ingest per 64-k block drops from 16 + BN / 8 KB to 16 + BN / 16 KB, which is what
// bounds the one-CTA kernel.  Rank 0 of the pair issues all MMAs (M = 256) and owns the `full` barriers, on which both
// CTAs' copies count; its commits arrive on the `empty` / accumulator-ready barriers of both CTAs; the epilogue warps
// of both CTAs release an accumulator on rank 0's barrier.  Whole tiles only.
template <int EPI, int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_pair_kernel(const __grid_constant__ GemmParams p) {
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE = A_BYTES + B_BYTES;
  constexpr int NST = RING_BYTES / STAGE;
  constexpr int TCOLS = 2 * BN;
  static_assert(NST >= 4 && TCOLS <= 512 && TCOLS >= 32 && (TCOLS & (TCOLS - 1)) == 0, "ring / TMEM capacity");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bars[2 * NST + 4];
  __shared__ uint32_t s_tmem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const uint32_t ring = ptx::smem_u32(smem);
  const uint32_t full = ptx::smem_u32(bars), empty = full + 8 * NST, tfull = empty + 8 * NST, tempty = tfull + 16;
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) { ptx::mbar_init(full + 8 * i, 1); ptx::mbar_init(empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { ptx::mbar_init(tfull + 8 * i, 1); ptx::mbar_init(tempty + 8 * i, 256); }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_shared();
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(&s_tmem), TCOLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();               // the partner's barriers exist before anything arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem = s_tmem;
  const int m_pairs = (p.m_tiles + 1) / 2, ntiles = p.n_tiles * m_pairs;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const bool leader = ptx::elect_one();
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();

  if (warp == 0) {
    // ---- producer (both CTAs): own token rows of A, own half of the tile's weight rows; bytes count on rank 0's barrier
    uint32_t slot = 0, par = 0;
    for (int tile = pair; tile < ntiles; tile += npairs) {
      const int nt = tile / m_pairs, mt = (tile % m_pairs) * 2 + (int)rank;
      const CUtensorMap* mb;
      int rb0;
      if (EPI == EPI_GEGLU) {          // rank 0: the tile's 128 gate rows, rank 1: the matching 128 up rows
        mb = rank ? &p.b1 : &p.b0;
        rb0 = p.layer * FFN + nt * (BN / 2);
      } else {
        mb = &p.b0;
        rb0 = p.layer * H + nt * BN + (int)rank * (BN / 2);
      }
      for (int kb = 0; kb < p.kblocks; ++kb) {
        if (!wait_bar(p.status, p.wait_limit, empty + 8 * slot, par ^ 1, 1)) goto done;
        if (leader) {
          const uint32_t bar = ptx::map_to_rank(full + 8 * slot, 0), dst = ring + slot * STAGE;
          if (rank == 0) ptx::mbar_expect_tx(full + 8 * slot, 2 * STAGE);
          ptx::tma_load_2d_pair(dst, &p.a, bar, kb * BK, mt * BM);
          ptx::tma_load_2d_pair(dst + A_BYTES, mb, bar, kb * BK, rb0);
        }
        if (++slot == NST) { slot = 0; par ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: rank 0 only
    if (rank == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(2 * BM, BN);
      const uint64_t adesc0 = ptx::umma_smem_desc(ring), bdesc0 = ptx::umma_smem_desc(ring + A_BYTES);
      uint32_t slot = 0, par = 0, it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < ntiles; tile += npairs, ++it) {
        const uint32_t buf = it & 1;
        if (!wait_bar(p.status, p.wait_limit, tempty + 8 * buf, ((it >> 1) & 1) ^ 1, 2)) break;
        ptx::tc_fence_after();
        const uint32_t d = tmem + buf * BN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!wait_bar(p.status, p.wait_limit, full + 8 * slot, par, 3)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint64_t off = (uint64_t)(slot * (STAGE >> 4));
          if (leader) {
            asm volatile(
                "{\n.reg .pred p;\n.reg .b64 a1, a2, a3, b1, b2, b3;\n"
                "setp.ne.b32 p, %4, 0;\n"
                "add.u64 a1, %1, 2;\n add.u64 a2, %1, 4;\n add.u64 a3, %1, 6;\n"
                "add.u64 b1, %2, 2;\n add.u64 b2, %2, 4;\n add.u64 b3, %2, 6;\n"
                "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
                "tcgen05.mma.cta_group::2.kind::f16 [%0], a1, b1, %3, 1;\n"
                "tcgen05.mma.cta_group::2.kind::f16 [%0], a2, b2, %3, 1;\n"
                "tcgen05.mma.cta_group::2.kind::f16 [%0], a3, b3, %3, 1;\n}"
                ::"r"(d), "l"(adesc0 + off), "l"(bdesc0 + off), "r"(idesc), "r"(kb ? 1u : 0u) : "memory");
            ptx::umma_commit_pair(empty + 8 * slot);
          }
          if (++slot == NST) { slot = 0; par ^= 1; }
        }
        if (ok && leader) ptx::umma_commit_pair(tfull + 8 * buf);
      }
    }
  } else {
    // ---- epilogue (both CTAs): own 128 token rows of the pair's accumulator
    const int quad = warp & 3, row = quad * 32 + lane;
    const uint32_t tempty0 = ptx::map_to_rank(tempty, 0);
    uint32_t it = 0;
    for (int tile = pair; tile < ntiles; tile += npairs, ++it) {
      const int nt = tile / m_pairs, mt = (tile % m_pairs) * 2 + (int)rank;
      const uint32_t buf = it & 1;
      const int token = mt * BM + row;
      if (!wait_bar(p.status, p.wait_limit, tfull + 8 * buf, (it >> 1) & 1, 4)) break;
      ptx::tc_fence_after();
      epilogue_row<EPI, BN>(p, tmem + buf * BN + ((uint32_t)(quad * 32) << 16), nt, token, token < p.tokens);
      ptx::tc_fence_before();
      ptx::mbar_arrive_cluster(tempty0 + 8 * buf);
    }
  }
done:
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();               // neither CTA leaves (or frees tensor memory) while the other may still use it
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem, TCOLS);
  }
}

// Gemma RMSNorm (the reference's rms(x, weight, gemma=True), reference/pi05.py:178, 192): FP32 normalisation, scale by
// (1 + weight), one rounding to BF16.  One warp per token row of 2048.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                               __nv_bfloat16* __restrict__ out, int tokens) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();
  if (row >= tokens) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 xv[8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    xv[j] = xr[lane + 32 * j];
    const uint32_t ws[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float a = lo16(ws[e]), b = hi16(ws[e]); ss += a * a + b * b; }
  }
  for (int sh = 16; sh; sh >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, sh);
  const float rs = rsqrtf(ss * (1.0f / H) + EPS);
  uint4* orow = reinterpret_cast<uint4*>(out + (size_t)row * H);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint4 wv = wr[lane + 32 * j];
    const uint32_t xs[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o[e] = pack2(__fmul_rn(__fmul_rn(lo16(xs[e]), rs), __fadd_rn(1.0f, lo16(ws[e]))),
                   __fmul_rn(__fmul_rn(hi16(xs[e]), rs), __fadd_rn(1.0f, hi16(ws[e]))));
    orow[lane + 32 * j] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// positions = cumsum(valid) - 1 (reference/pi05.py:173): one block, a block-wide scan in chunks of 1024 tokens.
__global__ void positions_kernel(const uint8_t* __restrict__ valid, int tokens, int* __restrict__ positions) {
  __shared__ int warp_sum[32];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < tokens; base += 1024) {
    const int t = base + threadIdx.x;
    int v = t < tokens && valid[t] ? 1 : 0;
    for (int sh = 1; sh < 32; sh <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, sh); if (lane >= sh) v += u; }
    if (lane == 31) warp_sum[warp] = v;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sum[lane];
      for (int sh = 1; sh < 32; sh <<= 1) { const int u = __shfl_up_sync(0xffffffffu, w, sh); if (lane >= sh) w += u; }
      warp_sum[lane] = w;
    }
    __syncthreads();
    const int incl = v + (warp ? warp_sum[warp - 1] : 0) + carry;
    if (t < tokens) positions[t] = incl - 1;
    __syncthreads();
    if (threadIdx.x == 1023) carry = incl;
    __syncthreads();
  }
}

// The BF16 cos / sin of every (token, rotary index) (reference/pi05.py:218-229: FP32 inverse frequencies and phases).
__global__ void rope_table_kernel(const int* __restrict__ positions, int tokens, uint32_t* __restrict__ rope) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < tokens * 128; i += gridDim.x * blockDim.x) {
    const int t = i >> 7, j = i & 127;
    const float e = (float)(2 * j) / 256.0f;
    const float inv = 1.0f / (float)pow(10000.0, (double)e);
    const float phase = (float)positions[t] * inv;
    __nv_bfloat162 v = __floats2bfloat162_rn((float)cos((double)phase), (float)sin((double)phase));
    rope[i] = *reinterpret_cast<uint32_t*>(&v);
  }
}

__global__ void cast_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------------------------------- prefill attention
// 128 query rows per CTA (16 tokens x 8 heads, all sharing the one KV head) against every key of the layer, on the
// tcgen05 tensor cores, in two passes over the keys so that nothing ever has to be rescaled:
//   pass 1  S = Q K^T chunk by chunk (64 keys) into one of two TMEM buffers; the softmax threads (one per query row) read
//           their row and keep the maximum over the valid keys;
//   pass 2  S again; P = exp(S - max) (0 for masked keys) is rounded to BF16 and written to shared memory in the
//           K-major swizzled layout an MMA A operand has, the FP32 row sum is kept by the thread, and O += P V
//           accumulates in 256 TMEM columns with the values read as V^T [256 dims, keys] (written by the QKV epilogue),
//           so that both MMAs take K-major operands.  O / sum goes out as BF16.
// Scores are rounded to BF16 and scaled by 1/16 as the reference's BF16 matmul and scale do (reference/pi05.py:184-188).
// Warp 0 streams Q, the key chunks (the 256 dims of a token as four 64-dim segments, 128-byte swizzle) and the V^T
// chunks with TMA through two-stage rings; warp 1 issues the MMAs (S of chunk c + 1 before P V of chunk c, so that the
// tensor core works while chunk c's probabilities are being made); warps 2..5 are the softmax threads.
namespace pfa {
constexpr int TOK = 16, ROWS = 128, KCH = 64, STG = 2, THREADS_A = 192;
constexpr int Q_BYTES = ROWS * HD * 2;                        // four 64-dim blocks of [128 rows x 128 B]
constexpr int K_BYTES = KCH * HD * 2;                         // four 64-dim segments of [64 keys x 128 B]
constexpr int V_BYTES = HD * KCH * 2;                         // [256 dims x 64 keys]
constexpr int P_BYTES = ROWS * KCH * 2;                       // [128 rows x 64 keys]
constexpr int OFF_Q = 0, OFF_K = OFF_Q + Q_BYTES, OFF_V = OFF_K + STG * K_BYTES, OFF_P = OFF_V + STG * V_BYTES;
constexpr int SMEM_A = OFF_P + 2 * P_BYTES + 1024;
constexpr int TM_O = 0, TM_S = 256, TM_COLS = 512;            // TMEM columns: O [128 x 256], two S buffers [128 x 64]
constexpr int MASK_WORDS = 128;                               // validity bits of up to 4096 tokens
static_assert(SMEM_A <= 227 * 1024, "attention shared memory");

struct AttnParams {
  CUtensorMap qmap;                  // q as [tokens * 8 rows, 256 dims], box {64, 128}
  CUtensorMap kmap;                  // {64 dims, tokens, 4 segments, layers, 1}, box {64, 64, 4, 1, 1}
  CUtensorMap vtmap;                 // V^T of the layer [256 dims, tokens], box {64 keys, 256}
  const uint8_t* valid;              // [tokens]
  __nv_bfloat16* out;                // [tokens, 2048]
  int tokens, layer;
  unsigned int* status;
  long long wait_limit;
};

// Four K = 16 MMAs over one 64-k operand block (32-byte steps inside the 128-byte swizzle row).
__device__ __forceinline__ void umma_k64(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "add.u64 a1, %1, 2;\n add.u64 a2, %1, 4;\n add.u64 a3, %1, 6;\n"
      "add.u64 b1, %2, 2;\n add.u64 b2, %2, 4;\n add.u64 b3, %2, 6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, 1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, 1;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, 1;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(THREADS_A, 1) attention_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // barriers: q, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full[2], p_empty[2], o_full
  __shared__ uint64_t bars[20];
  __shared__ uint32_t s_tmem;
  __shared__ uint32_t s_mask[MASK_WORDS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int npc = (p.tokens + KCH - 1) / KCH;
  const uint32_t b0 = ptx::smem_u32(bars);
  const uint32_t q_full = b0, k_full = b0 + 8, k_empty = b0 + 24, v_full = b0 + 40, v_empty = b0 + 56;
  const uint32_t s_full = b0 + 72, s_empty = b0 + 88, p_full = b0 + 104, p_empty = b0 + 120, o_full = b0 + 136;
  if (tid == 0) {
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(k_full + 8 * i, 1); ptx::mbar_init(k_empty + 8 * i, 1);
      ptx::mbar_init(v_full + 8 * i, 1); ptx::mbar_init(v_empty + 8 * i, 1);
      ptx::mbar_init(s_full + 8 * i, 1); ptx::mbar_init(s_empty + 8 * i, 128);
      ptx::mbar_init(p_full + 8 * i, 128); ptx::mbar_init(p_empty + 8 * i, 1);
    }
    ptx::mbar_init(o_full, 1);
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_shared();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&s_tmem), TM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = s_tmem;
  const bool leader = ptx::elect_one();
  const uint32_t sbase = ptx::smem_u32(smem);
  ptx::grid_dep_launch();
  ptx::grid_dep_wait();

  if (warp == 0) {
    // ---- producer: Q once, the key chunks twice (pass 1, pass 2), the V^T chunks in pass 2
    if (leader) {
      ptx::mbar_expect_tx(q_full, Q_BYTES);
      for (int kb = 0; kb < 4; ++kb)
        ptx::tma_load_2d(sbase + OFF_Q + kb * (ROWS * 128), &p.qmap, q_full, kb * 64, blockIdx.x * ROWS);
    }
    for (int i = 0; i < 2 * npc; ++i) {
      const int c = i < npc ? i : i - npc, slot = i & 1;
      if (!wait_bar(p.status, p.wait_limit, k_empty + 8 * slot, ((i >> 1) & 1) ^ 1, 1)) break;
      if (leader) {
        ptx::mbar_expect_tx(k_full + 8 * slot, K_BYTES);
        ptx::tma_load_5d(sbase + OFF_K + slot * K_BYTES, &p.kmap, k_full + 8 * slot, 0, c * KCH, 0, p.layer, 0);
      }
      if (i >= npc) {
        const int vslot = c & 1;
        if (!wait_bar(p.status, p.wait_limit, v_empty + 8 * vslot, ((c >> 1) & 1) ^ 1, 2)) break;
        if (leader) {
          ptx::mbar_expect_tx(v_full + 8 * vslot, V_BYTES);
          ptx::tma_load_2d(sbase + OFF_V + vslot * V_BYTES, &p.vtmap, v_full + 8 * vslot, c * KCH, 0);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    const uint32_t idesc_s = ptx::umma_idesc_bf16(ROWS, KCH), idesc_o = ptx::umma_idesc_bf16(ROWS, HD);
    const uint64_t qdesc = ptx::umma_smem_desc(sbase + OFF_Q), kdesc = ptx::umma_smem_desc(sbase + OFF_K);
    const uint64_t vdesc = ptx::umma_smem_desc(sbase + OFF_V), pdesc = ptx::umma_smem_desc(sbase + OFF_P);
    bool ok = wait_bar(p.status, p.wait_limit, q_full, 0, 3);
    // S tile i (i counts through both passes) into S buffer i & 1 from key stage i & 1
    auto issue_s = [&](int i) -> bool {
      const int slot = i & 1;
      if (!wait_bar(p.status, p.wait_limit, k_full + 8 * slot, (i >> 1) & 1, 4)) return false;
      if (!wait_bar(p.status, p.wait_limit, s_empty + 8 * slot, ((i >> 1) & 1) ^ 1, 5)) return false;
      ptx::tc_fence_after();
      if (leader) {
        const uint32_t d = tmem + TM_S + slot * KCH;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
          umma_k64(d, qdesc + (uint64_t)(kb * (ROWS * 128 >> 4)), kdesc + (uint64_t)((slot * K_BYTES + kb * (KCH * 128)) >> 4),
                   idesc_s, kb ? 1u : 0u);
        ptx::umma_commit(k_empty + 8 * slot);
        ptx::umma_commit(s_full + 8 * slot);
      }
      return true;
    };
    // O += P V for chunk c of pass 2
    auto issue_pv = [&](int c) -> bool {
      const int slot = c & 1;
      if (!wait_bar(p.status, p.wait_limit, p_full + 8 * slot, (c >> 1) & 1, 6)) return false;
      if (!wait_bar(p.status, p.wait_limit, v_full + 8 * slot, (c >> 1) & 1, 7)) return false;
      ptx::tc_fence_after();
      if (leader) {
        umma_k64(tmem + TM_O, pdesc + (uint64_t)((slot * P_BYTES) >> 4), vdesc + (uint64_t)((slot * V_BYTES) >> 4), idesc_o,
                 c ? 1u : 0u);
        ptx::umma_commit(v_empty + 8 * slot);
        ptx::umma_commit(p_empty + 8 * slot);
      }
      return true;
    };
    for (int i = 0; ok && i < npc; ++i) ok = issue_s(i);
    for (int c = 0; ok && c < npc; ++c) {
      ok = issue_s(npc + c);
      if (ok && c >= 1) ok = issue_pv(c - 1);
    }
    if (ok) ok = issue_pv(npc - 1);
    if (ok && leader) ptx::umma_commit(o_full);
  } else {
    // ---- softmax threads: thread = query row (TMEM lane); warp w may touch lanes 32 (w % 4) .. only
    const int quad = warp & 3, row = quad * 32 + lane, st = tid - 64;
    // validity bits of all keys, once
    for (int w = (st >> 5); w < MASK_WORDS; w += 4) {
      const int t = w * 32 + lane;
      const unsigned bits = __ballot_sync(0xffffffffu, t < p.tokens && p.valid[t] != 0);
      if (lane == 0) s_mask[w] = bits;
      if (w * 32 >= p.tokens) break;
    }
    ptx::named_bar_sync(1, 128);
    const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
    bool ok = true;
    float mraw = -INFINITY;
    // pass 1: the row maximum over the valid keys
    for (int i = 0; ok && i < npc; ++i) {
      const int slot = i & 1;
      if (!wait_bar(p.status, p.wait_limit, s_full + 8 * slot, (i >> 1) & 1, 8)) { ok = false; break; }
      ptx::tc_fence_after();
      uint32_t r0[32], r1[32];
      ptx::tmem_ld_32x32(trow + TM_S + slot * KCH, r0);
      ptx::tmem_ld_32x32(trow + TM_S + slot * KCH + 32, r1);
      ptx::tmem_wait_ld();
      ptx::tc_fence_before();
      ptx::mbar_arrive(s_empty + 8 * slot);
      // (rounding to BF16 and the scale are monotonic: the maximum of the raw scores is rounded once, after the pass)
      const uint32_t m0 = s_mask[2 * i], m1 = s_mask[2 * i + 1];
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if ((m0 & m1) == 0xffffffffu) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(r0[j]));
          mx[j & 3] = fmaxf(mx[j & 3], __uint_as_float(r1[j]));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          mx[j & 3] = fmaxf(mx[j & 3], (m0 & (1u << j)) ? __uint_as_float(r0[j]) : -INFINITY);
          mx[j & 3] = fmaxf(mx[j & 3], (m1 & (1u << j)) ? __uint_as_float(r1[j]) : -INFINITY);
        }
      }
      mraw = fmaxf(mraw, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])));
    }
    const float m = fmaxf(rb(mraw) * 0.0625f, -1e30f);
    // pass 2: probabilities
    float l = 0.f;
    constexpr float SCALE_LOG2E = 0.0625f * 1.4426950408889634f;
    const float mneg = -m * 1.4426950408889634f;
    const uint32_t prow = sbase + OFF_P + row * 128, psw = row & 7;
    for (int c = 0; ok && c < npc; ++c) {
      const int i = npc + c, slot = i & 1, pslot = c & 1;
      if (!wait_bar(p.status, p.wait_limit, s_full + 8 * slot, (i >> 1) & 1, 9)) { ok = false; break; }
      ptx::tc_fence_after();
      uint32_t r0[32], r1[32];
      ptx::tmem_ld_32x32(trow + TM_S + slot * KCH, r0);
      ptx::tmem_ld_32x32(trow + TM_S + slot * KCH + 32, r1);
      ptx::tmem_wait_ld();
      ptx::tc_fence_before();
      ptx::mbar_arrive(s_empty + 8 * slot);
      const uint32_t m0 = s_mask[2 * c], m1 = s_mask[2 * c + 1];
      // p = exp(bf16(s) / 16 - m) as one FMA and one ex2 per score; every score is computed, masked ones are replaced
      // afterwards, so that the 64 chains stay independent of each other
      uint32_t pk[32];
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      const bool all_valid = (m0 & m1) == 0xffffffffu;
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const uint32_t s0 = pack2(__uint_as_float(r0[j]), __uint_as_float(r0[j + 1]));
        const uint32_t s1 = pack2(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1]));
        float a = ptx::ex2_approx(fmaf(lo16(s0), SCALE_LOG2E, mneg)), b = ptx::ex2_approx(fmaf(hi16(s0), SCALE_LOG2E, mneg));
        float e = ptx::ex2_approx(fmaf(lo16(s1), SCALE_LOG2E, mneg)), f = ptx::ex2_approx(fmaf(hi16(s1), SCALE_LOG2E, mneg));
        if (!all_valid) {
          a = (m0 & (1u << j)) ? a : 0.f; b = (m0 & (2u << j)) ? b : 0.f;
          e = (m1 & (1u << j)) ? e : 0.f; f = (m1 & (2u << j)) ? f : 0.f;
        }
        ls[(j >> 1) & 3] += (a + b) + (e + f);
        pk[j >> 1] = pack2(a, b);
        pk[16 + (j >> 1)] = pack2(e, f);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      // the P buffer is free once the P V of chunk c - 2 has read it
      if (!wait_bar(p.status, p.wait_limit, p_empty + 8 * pslot, ((c >> 1) & 1) ^ 1, 10)) { ok = false; break; }
      const uint32_t dst = prow + pslot * P_BYTES;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)   // 16-byte piece ch of the row sits at piece ch ^ (row & 7) of its 128-byte line
        ptx::st_shared_v4(dst + (((uint32_t)ch ^ psw) << 4), pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
      ptx::fence_proxy_async_shared();
      ptx::mbar_arrive(p_full + 8 * pslot);
    }
    // ---- O / l -> BF16: row = token_local * 8 + head, so a row's 256 dims are contiguous in [tokens, 2048]
    if (ok && wait_bar(p.status, p.wait_limit, o_full, 0, 11)) {
      ptx::tc_fence_after();
      const float il = 1.0f / l;
      const int token = blockIdx.x * TOK + (row >> 3);
      __nv_bfloat16* orow = p.out + (size_t)token * QD + (row & 7) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(trow + TM_O + c0, r);
        ptx::tmem_wait_ld();
        if (token < p.tokens) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c0);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_uint4(pack2(__uint_as_float(r[8 * j]) * il, __uint_as_float(r[8 * j + 1]) * il),
                                pack2(__uint_as_float(r[8 * j + 2]) * il, __uint_as_float(r[8 * j + 3]) * il),
                                pack2(__uint_as_float(r[8 * j + 4]) * il, __uint_as_float(r[8 * j + 5]) * il),
                                pack2(__uint_as_float(r[8 * j + 6]) * il, __uint_as_float(r[8 * j + 7]) * il));
        }
      }
      ptx::tc_fence_before();
    }
  }
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, TM_COLS);
  }
}
}  // namespace pfa

}  // namespace pf

// =========================================================================================== host side
struct pi05_prefill {
  int device = 0, sms = 0, max_tokens = 0;
  const void* weights[PI05_PREFILL_NUM_WEIGHTS] = {};
  uint8_t* ws = nullptr;
  size_t ws_bytes = 0;
  bool bound = false;
  bool overlap = PI05_PREFILL_OVERLAP != 0;   // launch each kernel so that its set-up overlaps the tail of the one before
  long long wait_limit = 4000000000ll;
  std::string last_error;
  // workspace offsets
  size_t off_status, off_x, off_n, off_q, off_mixed, off_act, off_rope, off_pos, off_vt, off_partial;
  int vt_stride = 0;
  unsigned int sk_epoch = 0;        // stream-K launches of the current prefill so far
};

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encoder() {
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

// {inner = K, rows} BF16 row-major, box {64 k, box_rows}, 128-byte swizzle; rows beyond `rows` read as zeros.
bool map_2d(CUtensorMap* m, const void* base, uint64_t inner, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {inner * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The layer's V^T [256 dims, tokens] with rows `stride` elements apart: box {64 keys, 256 dims}; keys at and beyond
// `tokens` read as zeros.
bool map_vt(CUtensorMap* m, const void* base, uint64_t tokens, uint64_t stride) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  cuuint64_t dims[2] = {tokens, 256};
  cuuint64_t strides[1] = {stride * 2};
  cuuint32_t box[2] = {64, 256};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Keys / values of all layers as the attention's tiled copies read them: {64 dims, tokens, 4 segments, layers, 1}.
bool map_kv(CUtensorMap* m, const void* base, uint64_t tokens) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  cuuint64_t dims[5] = {64, tokens, 4, (cuuint64_t)pf::LAYERS, 1};
  cuuint64_t strides[4] = {256 * 2, 64 * 2, tokens * 256 * 2, (cuuint64_t)pf::LAYERS * tokens * 256 * 2};
  cuuint32_t box[5] = {64, 64, 4, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Guard {
  int prev = -1;
  bool ok;
  explicit Guard(int dev) { if (cudaGetDevice(&prev) != cudaSuccess) prev = -1; ok = cudaSetDevice(dev) == cudaSuccess; }
  ~Guard() { if (prev >= 0) cudaSetDevice(prev); }
};

size_t up(size_t v) { return (v + 255) / 256 * 256; }
constexpr size_t CONTROL_BYTES = 256 + 1024 * 4;

// Launch with programmatic stream serialisation: the kernel may begin (set up its barriers and tensor memory) while the
// kernel before it in the stream drains; it reads nothing that kernel wrote before its grid_dep_wait.
// `pairs`: launch the grid as clusters of two CTAs.
template <typename... Params, typename... Args>
cudaError_t launch_after(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool overlap,
                         bool pairs, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (overlap) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (pairs) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = 2; at[n].val.clusterDim.y = 1; at[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = at; cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// How a prefill of `tokens` tokens is launched on a GPU of `sms` SMs: the decisions pi05_prefill_run takes and
// pi05_prefill_plan reports.
struct PrefillPlan {
  int m_tiles;        // 128-token tiles
  bool pairs;         // gate/up, down and O projections on CTA pairs (256-token tiles)
  bool sk_down;       // down projection as a stream-K launch of 128 x 256 tiles
  int down_tiles, down_kblocks, down_ctas;
};

PrefillPlan plan_prefill(int sms, int tokens) {
  PrefillPlan pl;
  pl.m_tiles = (tokens + pf::BM - 1) / pf::BM;
  // The down projection (K = 16384) as whole 128 x 128 tiles when those fill more than half of the SMs (measured at 968
  // tokens: 4.13 against 4.43 ms per prefill), as a stream-K launch of 128 x 256 tiles for shorter prompts (256 tokens: 2.43
  // against 2.71 ms), where whole tiles would leave most SMs without work for the longest GEMM of the layer.
  pl.sk_down = pl.m_tiles * (pf::H / 128) * 2 <= sms;
  // CTA pairs work on 256 tokens at a time: with a single tile of tokens the second CTA of every pair would idle.  Measured
  // at 968 tokens, ms per prefill: no pairs 4.15, gate/up on pairs 3.95, + down projection 3.73, + O projection 3.73-3.77.
  pl.pairs = pl.m_tiles >= 2;
  pl.down_kblocks = pf::FFN / pf::BK;
  pl.down_tiles = pl.m_tiles * (pf::H / 256);
  const long long units = (long long)pl.down_tiles * pl.down_kblocks;
  pl.down_ctas = units < sms ? (int)units : sms;
  return pl;
}

template <int EPI, int BN, bool SK>
cudaError_t launch_gemm(pi05_prefill* h, pf::GemmParams& gp, cudaStream_t stream) {
  static bool attr_set[64] = {};
  if (!attr_set[h->device]) {
    cudaError_t e = cudaFuncSetAttribute(pf::gemm_kernel<EPI, BN, SK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         pf::RING_BYTES + 1024);
    if (e != cudaSuccess) return e;
    attr_set[h->device] = true;
  }
  const long long tiles = (long long)gp.n_tiles * gp.m_tiles, work = SK ? tiles * gp.kblocks : tiles;
  const int grid = work < h->sms ? (int)work : h->sms;
  if (SK) gp.sk_epoch = ++h->sk_epoch;
  return launch_after(pf::gemm_kernel<EPI, BN, SK>, dim3(grid), dim3(pf::GEMM_THREADS), pf::RING_BYTES + 1024, stream,
                      h->overlap, false, gp);
}

// The same GEMM on CTA pairs: tiles of 256 tokens x BN features, grid = an even number of CTAs.
template <int EPI, int BN>
cudaError_t launch_gemm_pair(pi05_prefill* h, pf::GemmParams& gp, cudaStream_t stream) {
  static bool attr_set[64] = {};
  if (!attr_set[h->device]) {
    cudaError_t e = cudaFuncSetAttribute(pf::gemm_pair_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         pf::RING_BYTES + 1024);
    if (e != cudaSuccess) return e;
    attr_set[h->device] = true;
  }
  const int pair_tiles = gp.n_tiles * ((gp.m_tiles + 1) / 2), pairs = h->sms / 2;
  const int grid = 2 * (pair_tiles < pairs ? pair_tiles : pairs);
  return launch_after(pf::gemm_pair_kernel<EPI, BN>, dim3(grid), dim3(pf::GEMM_THREADS), pf::RING_BYTES + 1024, stream,
                      h->overlap, true, gp);
}

}  // namespace

extern "C" {

int pi05_prefill_create(int device, int max_tokens, pi05_prefill_t* out) {
  if (!out) return PI05_ERR_ARGUMENT;
  *out = nullptr;
  if (device < 0 || device >= 64 || max_tokens < 1 || max_tokens > 4096) return PI05_ERR_ARGUMENT;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { cudaGetLastError(); return PI05_ERR_NO_DEVICE; }
  if (device >= ndev) return PI05_ERR_ARGUMENT;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); return PI05_ERR_NO_DEVICE; }
  if (prop.major != 10) return PI05_ERR_NO_DEVICE;
  pi05_prefill* h = new (std::nothrow) pi05_prefill();
  if (!h) return PI05_ERR_ARGUMENT;
  h->device = device;
  h->sms = prop.multiProcessorCount;
  h->max_tokens = max_tokens;
  const size_t P = (size_t)(max_tokens + 1) / 2 * 2;      // the attention writes token pairs
  size_t off = 0;
  auto add = [&](size_t bytes) { const size_t at = off; off = up(off + bytes); return at; };
  h->off_status = add(CONTROL_BYTES);   // status words, then one stream-K flag per CTA
  h->off_x = add(P * pf::H * 2);
  h->off_n = add(P * pf::H * 2);
  h->off_q = add(P * QD * 2);
  h->off_mixed = add(P * QD * 2);
  h->off_act = add(P * (size_t)pf::FFN * 2);
  h->off_rope = add(P * 128 * 4);
  h->off_pos = add(P * 4);
  h->vt_stride = (max_tokens + 63) / 64 * 64;
  h->off_vt = add((size_t)HD * h->vt_stride * 2);
  h->off_partial = add((size_t)h->sms * pf::BM * 256 * 4);
  h->ws_bytes = off;
  *out = h;
  return PI05_OK;
}

int pi05_prefill_workspace_bytes(pi05_prefill_t h, size_t* bytes) {
  if (!h || !bytes) return PI05_ERR_ARGUMENT;
  *bytes = h->ws_bytes;
  return PI05_OK;
}

const char* pi05_prefill_last_error(pi05_prefill_t h) { return h ? h->last_error.c_str() : "bad handle"; }

int pi05_prefill_bind(pi05_prefill_t h, const void* const weights[PI05_PREFILL_NUM_WEIGHTS], void* workspace,
                      size_t workspace_bytes) {
  if (!h || !weights || !workspace) return PI05_ERR_ARGUMENT;
  if (workspace_bytes < h->ws_bytes || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    h->last_error = "workspace too small or not 256-byte aligned";
    return PI05_ERR_ARGUMENT;
  }
  for (int i = 0; i < PI05_PREFILL_NUM_WEIGHTS; ++i) {
    if (!weights[i] || (reinterpret_cast<uintptr_t>(weights[i]) & 15)) {
      h->last_error = "weight " + std::to_string(i) + " is null or not 16-byte aligned";
      return PI05_ERR_ARGUMENT;
    }
    h->weights[i] = weights[i];
  }
  h->ws = static_cast<uint8_t*>(workspace);
  h->bound = true;
  return PI05_OK;
}

int pi05_prefill_run(pi05_prefill_t h, const void* embeddings, const void* valid, int tokens, void* keys, void* values,
                     int n_layers, void* stream_) {
  if (!h || !embeddings || !valid || !keys || !values) return PI05_ERR_ARGUMENT;
  if (!h->bound) return PI05_ERR_NOT_BOUND;
  if (tokens < 1 || tokens > h->max_tokens || n_layers < 1 || n_layers > pf::LAYERS) return PI05_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(embeddings) & 15) || (reinterpret_cast<uintptr_t>(keys) & 15) ||
      (reinterpret_cast<uintptr_t>(values) & 15)) {
    h->last_error = "embeddings, keys and values must be 16-byte aligned";
    return PI05_ERR_ARGUMENT;
  }
  Guard guard(h->device);
  if (!guard.ok) return PI05_ERR_CUDA;
  cudaStream_t stream = (cudaStream_t)stream_;
  const int P = tokens;
  auto ptr = [&](size_t off) { return h->ws + off; };
  __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(ptr(h->off_x));
  __nv_bfloat16* nrm = reinterpret_cast<__nv_bfloat16*>(ptr(h->off_n));
  __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(ptr(h->off_q));
  __nv_bfloat16* mixed = reinterpret_cast<__nv_bfloat16*>(ptr(h->off_mixed));
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(ptr(h->off_act));
  uint32_t* rope = reinterpret_cast<uint32_t*>(ptr(h->off_rope));
  int* pos = reinterpret_cast<int*>(ptr(h->off_pos));
  unsigned int* status = reinterpret_cast<unsigned int*>(ptr(h->off_status));
  __nv_bfloat16* vt = reinterpret_cast<__nv_bfloat16*>(ptr(h->off_vt));
  const __nv_bfloat16* const* w = reinterpret_cast<const __nv_bfloat16* const*>(h->weights);
  enum { LN1 = 0, LN2, LQ, LK, LV, LO, LG, LU, LD };
  __nv_bfloat16* K = static_cast<__nv_bfloat16*>(keys);
  __nv_bfloat16* V = static_cast<__nv_bfloat16*>(values);

  h->sk_epoch = 0;
  cudaError_t e = cudaMemsetAsync(status, 0, CONTROL_BYTES, stream);
  if (e != cudaSuccess) { h->last_error = cudaGetErrorString(e); return PI05_ERR_CUDA; }
  pf::cast_copy_kernel<<<h->sms, 256, 0, stream>>>(static_cast<const uint4*>(embeddings), reinterpret_cast<uint4*>(x),
                                                   (size_t)P * pf::H * 2 / 16);
  pf::positions_kernel<<<1, 1024, 0, stream>>>(static_cast<const uint8_t*>(valid), P, pos);
  pf::rope_table_kernel<<<h->sms, 256, 0, stream>>>(pos, P, rope);

  // tensor maps: activations (rows = tokens, zero beyond), weights (all layers stacked), keys / values for the attention
  pf::GemmParams base;
  memset(&base, 0, sizeof base);
  base.tokens = P; base.m_tiles = (P + pf::BM - 1) / pf::BM;
  base.x = x; base.act = act; base.q = q; base.rope = rope; base.status = status; base.wait_limit = h->wait_limit;
  base.vt = vt; base.vt_stride = h->vt_stride;
  base.sk_partial = reinterpret_cast<float*>(ptr(h->off_partial));
  base.sk_flags = status + 64;
  CUtensorMap a_n, a_mixed, a_act, wq, wk, wv, wo, wg, wu, wd, wd64, kmap, qmap, vtmap;
  bool ok = map_2d(&a_n, nrm, pf::H, P, pf::BM) && map_2d(&a_mixed, mixed, QD, P, pf::BM) &&
            map_2d(&a_act, act, pf::FFN, P, pf::BM) &&
            map_2d(&wq, w[LQ], pf::H, (uint64_t)pf::LAYERS * QD, 128) && map_2d(&wk, w[LK], pf::H, (uint64_t)pf::LAYERS * HD, 128) &&
            map_2d(&wv, w[LV], pf::H, (uint64_t)pf::LAYERS * HD, 128) && map_2d(&wo, w[LO], QD, (uint64_t)pf::LAYERS * pf::H, 64) &&
            map_2d(&wg, w[LG], pf::H, (uint64_t)pf::LAYERS * pf::FFN, 128) && map_2d(&wu, w[LU], pf::H, (uint64_t)pf::LAYERS * pf::FFN, 128) &&
            map_2d(&wd, w[LD], pf::FFN, (uint64_t)pf::LAYERS * pf::H, 128) &&
            map_2d(&wd64, w[LD], pf::FFN, (uint64_t)pf::LAYERS * pf::H, 64) && map_kv(&kmap, K, P) && map_2d(&qmap, q, HD, (uint64_t)P * 8, 128) &&
            map_vt(&vtmap, vt, P, h->vt_stride);
  if (!ok) { h->last_error = "cuTensorMapEncodeTiled failed"; return PI05_ERR_CUDA; }

  static bool att_attr[64] = {};
  if (!att_attr[h->device]) {
    e = cudaFuncSetAttribute(pf::pfa::attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pf::pfa::SMEM_A);
    if (e != cudaSuccess) { h->last_error = cudaGetErrorString(e); return PI05_ERR_CUDA; }
    att_attr[h->device] = true;
  }
  pf::pfa::AttnParams ap;
  memset(&ap, 0, sizeof ap);
  ap.qmap = qmap; ap.kmap = kmap; ap.vtmap = vtmap;
  ap.valid = static_cast<const uint8_t*>(valid); ap.out = mixed;
  ap.tokens = P; ap.status = status; ap.wait_limit = h->wait_limit;

  const int norm_blocks = (P + 7) / 8;
  const PrefillPlan plan = plan_prefill(h->sms, P);
  const bool sk_down = plan.sk_down, pairs_pay = plan.pairs;
  for (int l = 0; l < n_layers; ++l) {
    if ((e = launch_after(pf::rmsnorm_kernel, dim3(norm_blocks), dim3(256), 0, stream, h->overlap && l > 0, false,
                          (const __nv_bfloat16*)x, w[LN1] + (size_t)l * pf::H, nrm, P)) != cudaSuccess) break;
    {
      pf::GemmParams gp = base;
      gp.a = a_n; gp.b0 = gp.b1 = wq; gp.b2 = wk; gp.b3 = wv;
      gp.kblocks = pf::H / pf::BK; gp.n_tiles = 10; gp.layer = l;
      gp.k = K + (size_t)l * P * HD; gp.v = V + (size_t)l * P * HD;
      if ((e = launch_gemm<pf::EPI_QKV, 256, false>(h, gp, stream)) != cudaSuccess) break;
    }
    ap.layer = l;
    if ((e = launch_after(pf::pfa::attention_kernel, dim3((P + pf::pfa::TOK - 1) / pf::pfa::TOK), dim3(pf::pfa::THREADS_A),
                          pf::pfa::SMEM_A, stream, h->overlap, false, ap)) != cudaSuccess) break;
    {
      pf::GemmParams gp = base;
      gp.a = a_mixed; gp.b0 = gp.b1 = wo;
      gp.kblocks = QD / pf::BK; gp.n_tiles = pf::H / 128; gp.layer = l;
      e = pairs_pay ? launch_gemm_pair<pf::EPI_RESID, 128>(h, gp, stream)
                                         : launch_gemm<pf::EPI_RESID, 128, false>(h, gp, stream);
      if (e != cudaSuccess) break;
    }
    if (l + 1 == n_layers) break;          // the last MLP does not affect any cached key or value
    if ((e = launch_after(pf::rmsnorm_kernel, dim3(norm_blocks), dim3(256), 0, stream, h->overlap, false,
                          (const __nv_bfloat16*)x, w[LN2] + (size_t)l * pf::H, nrm, P)) != cudaSuccess) break;
    {
      pf::GemmParams gp = base;
      gp.a = a_n; gp.b0 = wg; gp.b1 = wu;
      gp.kblocks = pf::H / pf::BK; gp.n_tiles = pf::FFN / 128; gp.layer = l;
      e = pairs_pay ? launch_gemm_pair<pf::EPI_GEGLU, 256>(h, gp, stream)
                                             : launch_gemm<pf::EPI_GEGLU, 256, false>(h, gp, stream);
      if (e != cudaSuccess) break;
    }
    {
      pf::GemmParams gp = base;
      gp.a = a_act; gp.b0 = gp.b1 = sk_down ? wd : wd64;
      gp.kblocks = pf::FFN / pf::BK; gp.n_tiles = pf::H / (sk_down ? 256 : 128); gp.layer = l;
      e = sk_down ? launch_gemm<pf::EPI_RESID, 256, true>(h, gp, stream)
          : pairs_pay ? launch_gemm_pair<pf::EPI_RESID, 128>(h, gp, stream)
                                             : launch_gemm<pf::EPI_RESID, 128, false>(h, gp, stream);
      if (e != cudaSuccess) break;
    }
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) { h->last_error = std::string("kernel launch: ") + cudaGetErrorString(e); return PI05_ERR_CUDA; }
  return PI05_OK;
}

int pi05_prefill_plan(int sms, int tokens, int cta, int info[PI05_PREFILL_PLAN_INFO], int* segments, int capacity, int* count) {
  if (sms < 2 || sms > 1024 || tokens < 1 || tokens > 4096 || !info || !count || capacity < 0 || (capacity && !segments))
    return PI05_ERR_ARGUMENT;
  const PrefillPlan pl = plan_prefill(sms, tokens);
  info[0] = pl.m_tiles; info[1] = pl.pairs; info[2] = pl.sk_down;
  info[3] = pl.sk_down ? pl.down_tiles : 0; info[4] = pl.sk_down ? pl.down_kblocks : 0; info[5] = pl.sk_down ? pl.down_ctas : 0;
  *count = 0;
  if (!pl.sk_down) return PI05_OK;
  if (cta < 0 || cta >= pl.down_ctas) return PI05_ERR_ARGUMENT;
  pf::Segments<true> segs(pl.down_kblocks, pl.down_tiles, cta, pl.down_ctas);
  int tile, kb0, kb1;
  while (segs.next(tile, kb0, kb1)) {
    if (*count < capacity) { segments[3 * *count] = tile; segments[3 * *count + 1] = kb0; segments[3 * *count + 2] = kb1; }
    ++*count;
  }
  return PI05_OK;
}

int pi05_prefill_status(pi05_prefill_t h, void* stream, int* code, int* where) {
  if (!h || !code || !where) return PI05_ERR_ARGUMENT;
  if (!h->ws) return PI05_ERR_NOT_BOUND;
  Guard guard(h->device);
  if (!guard.ok) return PI05_ERR_CUDA;
  unsigned int st[2] = {0, 0};
  cudaError_t e = cudaMemcpyAsync(st, h->ws + h->off_status, sizeof st, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) { h->last_error = cudaGetErrorString(e); return PI05_ERR_CUDA; }
  *code = (int)st[0];
  *where = (int)st[1];
  return st[0] ? PI05_ERR_DEVICE_TIMEOUT : PI05_OK;
}

int pi05_prefill_destroy(pi05_prefill_t h) {
  if (!h) return PI05_ERR_ARGUMENT;
  delete h;
  return PI05_OK;
}

}  // extern "C"
