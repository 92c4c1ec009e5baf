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
//     RoPE and the scatter into q / k / v, GeGLU, or the residual add;
//   * a row kernel for the Gemma RMSNorm, a table kernel for the RoPE factors;
//   * attention by the chunk engine's own attention code (16 query rows = 2 tokens x 8 heads against 64-key chunks
//     staged by tiled TMA copies, online softmax), driven by a small wrapper kernel.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <new>
#include <string>

#include "../../include/pi05_b200.h"
#include "ptx_sm100.cuh"

#include "pi05_common.cuh"
using namespace pi05;

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
  const uint32_t* rope;            // [tokens][128]: cos BF16 | sin BF16 << 16
  unsigned int* status;
  long long wait_limit;
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

// out[tokens, N] = A[tokens, K] . W[N, K]^T with a fused epilogue; tile = 128 tokens x BN features.
template <int EPI, int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
  constexpr int NST = RING_BYTES / STAGE;
  constexpr int TCOLS = 2 * BN;
  static_assert(NST >= 4 && TCOLS <= 512, "ring / TMEM budget");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bars[2 * NST + 4];
  __shared__ uint32_t s_tmem;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ring = ptx::smem_u32(smem);
  const uint32_t full = ptx::smem_u32(bars), empty = full + 8 * NST, tfull = empty + 8 * NST, tempty = tfull + 16;
  if (tid == 0) {
    for (int i = 0; i < NST; ++i) { ptx::mbar_init(full + 8 * i, 1); ptx::mbar_init(empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { ptx::mbar_init(tfull + 8 * i, 1); ptx::mbar_init(tempty + 8 * i, 128); }
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

  if (warp == 0) {
    // ---- producer: both operands of every stage, tile after tile (consecutive tiles share the weight rows)
    uint32_t slot = 0, par = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
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
      for (int kb = 0; kb < p.kblocks; ++kb) {
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
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const uint32_t buf = it & 1;
      if (!wait_bar(p.status, p.wait_limit, tempty + 8 * buf, ((it >> 1) & 1) ^ 1, 2)) break;
      ptx::tc_fence_after();
      const uint32_t d = tmem + buf * BN;
      for (int kb = 0; kb < p.kblocks; ++kb) {
        if (!wait_bar(p.status, p.wait_limit, full + 8 * slot, par, 3)) { kb = p.kblocks; tile = ntiles; break; }
        const uint64_t off = (uint64_t)(slot * (STAGE >> 4));
        if (leader) umma_stage4(d, adesc0 + off, bdesc0 + off, idesc, kb ? 1u : 0u, empty + 8 * slot);
        if (++slot == NST) { slot = 0; par ^= 1; }
      }
      if (leader) ptx::umma_commit(tfull + 8 * buf);
    }
  } else {
    // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) ..; thread = token row of the tile
    const int quad = warp & 3, row = quad * 32 + lane;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int nt = tile / p.m_tiles, mt = tile % p.m_tiles;
      const uint32_t buf = it & 1;
      const int token = mt * BM + row;
      const bool live = token < p.tokens;
      if (!wait_bar(p.status, p.wait_limit, tfull + 8 * buf, (it >> 1) & 1, 4)) break;
      ptx::tc_fence_after();
      const uint32_t t0 = tmem + buf * BN + ((uint32_t)(quad * 32) << 16);
      if (EPI == EPI_RESID) {
        __nv_bfloat16* xr = p.x + (size_t)token * H + nt * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(t0 + c, r);
          ptx::tmem_wait_ld();
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(xr + c);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 old = dst[j];
              const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
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
            } else {
              // RoPE (reference/pi05.py:218-229 on BF16 tensors): x cos + rotate_half(x) sin, every product and the
              // sum rounded to BF16; dims c.. pair with dims 128 + c..
              const uint32_t* cs = p.rope + (size_t)token * 128 + c;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float a[2], b[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const uint32_t w = cs[2 * j + e];
                  const float co = lo16(w), si = hi16(w);
                  const float x1 = rb(__uint_as_float(r1[2 * j + e])), x2 = rb(__uint_as_float(r2[2 * j + e]));
                  a[e] = rb(rb(x1 * co) + rb(-x2 * si));
                  b[e] = rb(rb(x2 * co) + rb(x1 * si));
                }
                o1[j] = pack2(a[0], a[1]);
                o2[j] = pack2(b[0], b[1]);
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

// Gemma RMSNorm (the reference's rms(x, weight, gemma=True), reference/pi05.py:178, 192): FP32 normalisation, scale by
// (1 + weight), one rounding to BF16.  One warp per token row of 2048.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                               __nv_bfloat16* __restrict__ out, int tokens) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
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

// positions = cumsum(valid) - 1 (reference/pi05.py:173) and the BF16 cos / sin of every (token, rotary index)
// (reference/pi05.py:218-229: FP32 inverse frequencies and phases).  One block; the count is a serial scan by warp 0.
__global__ void rope_table_kernel(const uint8_t* __restrict__ valid, int tokens, uint32_t* __restrict__ rope, int* __restrict__ positions) {
  extern __shared__ int s_pos[];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int t = 0; t < tokens; ++t) { acc += valid[t] ? 1 : 0; s_pos[t] = acc - 1; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < tokens; i += blockDim.x) positions[i] = s_pos[i];
  for (int i = threadIdx.x; i < tokens * 128; i += blockDim.x) {
    const int t = i >> 7, j = i & 127;
    const float e = (float)(2 * j) / 256.0f;
    const float inv = 1.0f / (float)pow(10000.0, (double)e);
    const float phase = (float)s_pos[t] * inv;
    __nv_bfloat162 v = __floats2bfloat162_rn((float)cos((double)phase), (float)sin((double)phase));
    rope[i] = *reinterpret_cast<uint32_t*>(&v);
  }
}

__global__ void cast_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

}  // namespace pf

// The chunk engine's device code once more, for its attention (16 query rows against TMA-staged 64-key chunks with an
// online softmax): the prefill's attention is the same computation without suffix keys.
#ifndef PI05_QF_KEPT
#define PI05_QF_KEPT 8
#endif
namespace k_pf {
#define PI05_TRACE 0
#define PI05_BATCHED 0
#define PI05_GN 1
#define PI05_TP 0
#include "pi05_chunk_kernel.cuh"
#undef PI05_TRACE
#undef PI05_BATCHED
#undef PI05_GN
#undef PI05_TP

// Two tokens x eight heads per CTA against all keys of this layer (the prefix itself).  `q` holds the rotated queries.
__global__ void __launch_bounds__(THREADS, 1) prefill_attention_kernel(const __grid_constant__ Params p,
                                                                       const __nv_bfloat16* __restrict__ q, int layer) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int unit = blockIdx.x, tid = threadIdx.x;
  const Ctx c{p.ctrl, p.wait_limit, unit, 20u};
  if (tid == 0) {
    reinterpret_cast<int*>(smem + OFF_PAGETAB)[0] = 0;
    for (int j = 0; j < 2 * ATT_STAGES; ++j) ptx::mbar_init(ptx::smem_u32(smem + OFF_ATTBARS) + 8 * j, 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  AttBars bars;
  const int npc = (p.prefix + 63) / 64;
  AttChunkIssue issue{p, p.ob, c, smem, bars, layer, npc, 0, npc};     // no suffix chunk: the keys end with the prefix
  const int nearly = min(npc, ATT_STAGES);
  for (int j = 0; j < nearly; ++j) issue(j, j);
  {
    const int m = tid >> 4, d0 = (tid & 15) * 16, t = unit * 2 + (m >> 3);
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
    if (t < p.prefix) {
      const uint4* src = reinterpret_cast<const uint4*>(q + (size_t)t * QD + (m & 7) * HD + d0);
      a = src[0]; b = src[1];
    }
    const uint32_t dst = ptx::smem_u32(smem + OFF_QS) + (m * KV_STRIDE + d0) * 2;
    ptx::st_shared_v4(dst, a.x, a.y, a.z, a.w);
    ptx::st_shared_v4(dst + 16, b.x, b.y, b.z, b.w);
  }
  if (!attention_unit(p, p.ob, smem, unit, issue, 0, nearly, 0, false)) att_drain(c, smem, bars, 0);
}
}  // namespace k_pf

// =========================================================================================== host side
struct pi05_prefill {
  int device = 0, sms = 0, max_tokens = 0;
  const void* weights[PI05_PREFILL_NUM_WEIGHTS] = {};
  uint8_t* ws = nullptr;
  size_t ws_bytes = 0;
  bool bound = false;
  long long wait_limit = 4000000000ll;
  std::string last_error;
  // workspace offsets
  size_t off_status, off_x, off_n, off_q, off_mixed, off_act, off_rope, off_pos;
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

template <int EPI, int BN>
cudaError_t launch_gemm(pi05_prefill* h, pf::GemmParams& gp, cudaStream_t stream) {
  static bool attr_set[64] = {};
  if (!attr_set[h->device]) {
    cudaError_t e = cudaFuncSetAttribute(pf::gemm_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         pf::RING_BYTES + 1024);
    if (e != cudaSuccess) return e;
    attr_set[h->device] = true;
  }
  const int tiles = gp.n_tiles * gp.m_tiles;
  const int grid = tiles < h->sms ? tiles : h->sms;
  pf::gemm_kernel<EPI, BN><<<grid, pf::GEMM_THREADS, pf::RING_BYTES + 1024, stream>>>(gp);
  return cudaGetLastError();
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
  h->off_status = add(256);
  h->off_x = add(P * pf::H * 2);
  h->off_n = add(P * pf::H * 2);
  h->off_q = add(P * QD * 2);
  h->off_mixed = add(P * QD * 2);
  h->off_act = add(P * (size_t)pf::FFN * 2);
  h->off_rope = add(P * 128 * 4);
  h->off_pos = add(P * 4);
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
  const __nv_bfloat16* const* w = reinterpret_cast<const __nv_bfloat16* const*>(h->weights);
  enum { LN1 = 0, LN2, LQ, LK, LV, LO, LG, LU, LD };
  __nv_bfloat16* K = static_cast<__nv_bfloat16*>(keys);
  __nv_bfloat16* V = static_cast<__nv_bfloat16*>(values);

  cudaError_t e = cudaMemsetAsync(status, 0, 256, stream);
  if (e != cudaSuccess) { h->last_error = cudaGetErrorString(e); return PI05_ERR_CUDA; }
  pf::cast_copy_kernel<<<h->sms, 256, 0, stream>>>(static_cast<const uint4*>(embeddings), reinterpret_cast<uint4*>(x),
                                                   (size_t)P * pf::H * 2 / 16);
  pf::rope_table_kernel<<<1, 1024, (size_t)P * 4, stream>>>(static_cast<const uint8_t*>(valid), P, rope, pos);

  // tensor maps: activations (rows = tokens, zero beyond), weights (all layers stacked), keys / values for the attention
  pf::GemmParams base;
  memset(&base, 0, sizeof base);
  base.tokens = P; base.m_tiles = (P + pf::BM - 1) / pf::BM;
  base.x = x; base.act = act; base.q = q; base.rope = rope; base.status = status; base.wait_limit = h->wait_limit;
  CUtensorMap a_n, a_mixed, a_act, wq, wk, wv, wo, wg, wu, wd, kmap, vmap;
  bool ok = map_2d(&a_n, nrm, pf::H, P, pf::BM) && map_2d(&a_mixed, mixed, QD, P, pf::BM) &&
            map_2d(&a_act, act, pf::FFN, P, pf::BM) &&
            map_2d(&wq, w[LQ], pf::H, (uint64_t)pf::LAYERS * QD, 128) && map_2d(&wk, w[LK], pf::H, (uint64_t)pf::LAYERS * HD, 128) &&
            map_2d(&wv, w[LV], pf::H, (uint64_t)pf::LAYERS * HD, 128) && map_2d(&wo, w[LO], QD, (uint64_t)pf::LAYERS * pf::H, 64) &&
            map_2d(&wg, w[LG], pf::H, (uint64_t)pf::LAYERS * pf::FFN, 128) && map_2d(&wu, w[LU], pf::H, (uint64_t)pf::LAYERS * pf::FFN, 128) &&
            map_2d(&wd, w[LD], pf::FFN, (uint64_t)pf::LAYERS * pf::H, 64) && map_kv(&kmap, K, P) && map_kv(&vmap, V, P);
  if (!ok) { h->last_error = "cuTensorMapEncodeTiled failed"; return PI05_ERR_CUDA; }

  // the attention's parameter block (the chunk engine's own type): prefix = tokens, one page per "observation"
  static bool att_attr[64] = {};
  if (!att_attr[h->device]) {
    e = cudaFuncSetAttribute(k_pf::prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) { h->last_error = cudaGetErrorString(e); return PI05_ERR_CUDA; }
    att_attr[h->device] = true;
  }
  Params ap;
  memset(&ap, 0, sizeof ap);
  ap.maps.pk = ap.maps.pk_tail = kmap;
  ap.maps.pv = ap.maps.pv_tail = vmap;
  ap.ob.prefix_mask = static_cast<const uint8_t*>(valid);
  ap.ob.attn = mixed;
  ap.ctrl = status;
  ap.wait_limit = h->wait_limit;
  ap.prefix = P; ap.key_groups = 1; ap.row_groups = 1; ap.batch = 1;
  ap.pages_per_obs = 1; ap.page_tokens = P;
  ap.drop_event = -1; ap.poll_ns = 20;

  const int norm_blocks = (P + 7) / 8;
  for (int l = 0; l < n_layers; ++l) {
    pf::rmsnorm_kernel<<<norm_blocks, 256, 0, stream>>>(x, w[LN1] + (size_t)l * pf::H, nrm, P);
    {
      pf::GemmParams gp = base;
      gp.a = a_n; gp.b0 = gp.b1 = wq; gp.b2 = wk; gp.b3 = wv;
      gp.kblocks = pf::H / pf::BK; gp.n_tiles = 10; gp.layer = l;
      gp.k = K + (size_t)l * P * HD; gp.v = V + (size_t)l * P * HD;
      if ((e = launch_gemm<pf::EPI_QKV, 256>(h, gp, stream)) != cudaSuccess) break;
    }
    k_pf::prefill_attention_kernel<<<(P + 1) / 2, THREADS, SMEM_BYTES, stream>>>(ap, q, l);
    {
      pf::GemmParams gp = base;
      gp.a = a_mixed; gp.b0 = gp.b1 = wo;
      gp.kblocks = QD / pf::BK; gp.n_tiles = pf::H / 128; gp.layer = l;
      if ((e = launch_gemm<pf::EPI_RESID, 128>(h, gp, stream)) != cudaSuccess) break;
    }
    if (l + 1 == n_layers) break;          // the last MLP does not affect any cached key or value
    pf::rmsnorm_kernel<<<norm_blocks, 256, 0, stream>>>(x, w[LN2] + (size_t)l * pf::H, nrm, P);
    {
      pf::GemmParams gp = base;
      gp.a = a_n; gp.b0 = wg; gp.b1 = wu;
      gp.kblocks = pf::H / pf::BK; gp.n_tiles = pf::FFN / 128; gp.layer = l;
      if ((e = launch_gemm<pf::EPI_GEGLU, 256>(h, gp, stream)) != cudaSuccess) break;
    }
    {
      pf::GemmParams gp = base;
      gp.a = a_act; gp.b0 = gp.b1 = wd;
      gp.kblocks = pf::FFN / pf::BK; gp.n_tiles = pf::H / 128; gp.layer = l;
      if ((e = launch_gemm<pf::EPI_RESID, 128>(h, gp, stream)) != cudaSuccess) break;
    }
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) { h->last_error = std::string("kernel launch: ") + cudaGetErrorString(e); return PI05_ERR_CUDA; }
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
