// Prompt attention on the 5th-generation tensor cores (tcgen05) for head sizes 64 and 128:
// causal, optional sliding window, grouped heads, prompts of unequal lengths packed back to
// back.  Scores and the output accumulate in tensor memory; queries, keys, values come by TMA
// (128-byte swizzle) straight from the step's packed projection.
//
//   grid (heads, query tiles, sequences); a CTA owns 128 consecutive queries of one head.  Blocks
//   are handed out in index order, so all heads' longest tiles (the last queries) start first
//   and the short ones fill the tail.
//   Two CTAs share an SM (half of its shared memory, tensor memory and registers each), so one
//   CTA's softmax overlaps the other's MMAs and loads.
//   warp 4      TMA producer: the query tile once, then key and value tiles of 64 positions
//               into a two-deep ring.
//   warp 5      MMA issuer.  S = Q K^T  (128 x 64 x HEAD_DIM, both operands K-major) into one
//               of two score buffers in TMEM, so the scores of the next tile are computed while
//               the softmax of this one runs;  O += P V  (128 x HEAD_DIM x 64: P from shared
//               memory, V as an MN-major operand, i.e. exactly as the projection stores it).
//   warps 0-3   softmax, one query row per thread (a row of TMEM is one lane): read the row
//               of scores, mask, running maximum and sum in fp32, exponentials on the
//               special-function unit, P as bf16 into (swizzled) shared memory.  The output
//               is rescaled in TMEM only when a row's maximum has grown by more than 2^8 since
//               the value the exponentials refer to, which keeps P within bf16 range and makes
//               rescaling rare; the final division uses the same reference maximum, so the
//               result is the exact softmax.
//   Every mbarrier wait is bounded; on expiry the kernel records IERT_ERR_WAIT_EXPIRED, frees
//   its TMEM and returns.
//
// Visible keys of query i: j in [max(0, i - (W - 1)), i] (src/layers/attention.rs:364-368);
// formulas src/layers/attention.rs:357-415, src/ops/softmax.rs:11-25.
#include "common.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<64 or 128>"
#endif

#if HEAD_DIM == 64 || HEAD_DIM == 128

using namespace iert;
using namespace sm100;

namespace {

constexpr int HD = HEAD_DIM;
constexpr int NSUB = HD / 64;                  // 64-element (128-byte) column blocks of a head
constexpr int BM = 128, BN = 64;               // queries per CTA, keys per tile
constexpr int SUB_BYTES = BM * 128;            // a block of the query / probability tile: 128 rows x 128 bytes
constexpr int KV_SUB_BYTES = BN * 128;         // a block of a key / value tile: 64 rows x 128 bytes
constexpr int THREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr uint32_t TMEM_COLS = 256;            // S0 [0,64) S1 [64,128) O [128, 128 + HD): two CTAs share an SM
constexpr uint32_t O_COL = 128;

struct PrefillTcParams {
  __nv_bfloat16* out;         // [T, heads * HD]
  int heads, kv_heads, window;
  float scale_log2e;
  int* err;
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  return false;
}
// Packed fp32 pairs (one instruction for two values) and the three-input maximum of sm_100.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            PrefillTcParams p, IertBatchView b) {
  // No static shared memory in this kernel: the dynamic window starts at the block's base,
  // which is 1024-byte aligned as the swizzled tiles need (checked below).
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;                                       // NSUB blocks of 128 rows
  uint8_t* k_s = q_s + NSUB * SUB_BYTES;                     // 2 stages x NSUB blocks of 64 rows
  uint8_t* v_s = k_s + 2 * NSUB * KV_SUB_BYTES;              // 2 stages x NSUB blocks of 64 rows
  uint64_t* bars = (uint64_t*)(v_s + 2 * NSUB * KV_SUB_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* v_full = bars + 3;      // 2
  uint64_t* k_empty = bars + 5;     // 2: a key buffer is free once its score MMAs have finished
  uint64_t* v_empty = bars + 7;     // 2: a value buffer is free once its output MMAs have finished
  uint64_t* s_full = bars + 9;      // 2: the scores of a tile are in their buffer
  uint64_t* p_ready = bars + 11;    // 2: the probabilities of a tile are in their buffer (every softmax thread arrives)
  uint64_t* pv_done = bars + 13;    // 2: the output MMAs of a tile have finished
  uint32_t* tmem_slot = (uint32_t*)(bars + 15);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int s = blockIdx.z, head = blockIdx.x;
  if (b.slot_ids[s] < 0) return;
  if (smem_addr(smem) & 1023u) {                             // never expected; refuse rather than compute garbage
    if (threadIdx.x == 0) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
    return;
  }
  const int q_begin = b.cu_q[s], len = b.cu_q[s + 1] - q_begin;
  const int n_qt = (len + BM - 1) / BM;
  const int qt = n_qt - 1 - (int)blockIdx.y;                 // the longest tiles start first
  if (qt < 0) return;
  const int i0 = qt * BM;
  const int kvh = head / (p.heads / p.kv_heads);
  const int i_hi = min(len, i0 + BM) - 1;
  const int j_lo = p.window > 0 ? max(0, i0 - (p.window - 1)) : 0;
  const int kt_lo = j_lo / BN, kt_hi = i_hi / BN;
  const int n_tiles = kt_hi - kt_lo + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 128); mbar_init(&pv_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_kv);
  }
  if (warp == 5) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before (the set-up above overlapped it)

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int q_col = head * HD, k_col = (p.heads + kvh) * HD, v_col = (p.heads + p.kv_heads + kvh) * HD;
      mbar_expect_tx(q_full, NSUB * SUB_BYTES);
      for (int sb = 0; sb < NSUB; ++sb) tma_load_2d(q_s + sb * SUB_BYTES, &map_q, q_full, q_col + 64 * sb, q_begin + i0);
      // keys run one tile ahead of values: a key buffer frees up earlier (after the scores)
      auto load_k = [&](int it) -> bool {
        const int st = it & 1;
        if (!wait_bar(&k_empty[st], ((it >> 1) & 1) ^ 1, abort_flag)) return false;
        mbar_expect_tx(&k_full[st], NSUB * KV_SUB_BYTES);
        for (int sb = 0; sb < NSUB; ++sb)
          tma_load_2d(k_s + (st * NSUB + sb) * KV_SUB_BYTES, &map_kv, &k_full[st], k_col + 64 * sb,
                      q_begin + (kt_lo + it) * BN);
        return true;
      };
      auto load_v = [&](int it) -> bool {
        const int st = it & 1;
        if (!wait_bar(&v_empty[st], ((it >> 1) & 1) ^ 1, abort_flag)) return false;
        mbar_expect_tx(&v_full[st], NSUB * KV_SUB_BYTES);
        for (int sb = 0; sb < NSUB; ++sb)
          tma_load_2d(v_s + (st * NSUB + sb) * KV_SUB_BYTES, &map_kv, &v_full[st], v_col + 64 * sb,
                      q_begin + (kt_lo + it) * BN);
        return true;
      };
      ok = load_k(0);
      if (ok && n_tiles > 1) ok = load_k(1);
      for (int it = 0; ok && it < n_tiles; ++it) {
        ok = load_v(it);
        if (ok && it + 2 < n_tiles) ok = load_k(it + 2);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t IDESC_S = instr_desc_bf16(BM, BN);
      constexpr uint32_t IDESC_O = instr_desc_bf16_b_mn(BM, HD);
      // The MMAs of this thread run in the order they are issued, so a score buffer needs no barrier of
      // its own: the scores of tile it + 2 are issued after the output MMAs of tile it, which read the
      // probabilities that the softmax wrote over the scores of tile it.
      auto scores = [&](int it) -> bool {                    // S[it & 1] = Q K_it^T
        const int st = it & 1;
        if (!wait_bar(&k_full[st], (it >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t qa = smem_addr(q_s + (ks / 4) * SUB_BYTES) + (ks % 4) * 32;
          const uint32_t kb = smem_addr(k_s + (st * NSUB + ks / 4) * KV_SUB_BYTES) + (ks % 4) * 32;
          umma_bf16(tmem_base + st * BN, smem_desc_k128(qa), smem_desc_k128(kb), IDESC_S, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        return true;
      };
      if (!wait_bar(q_full, 0, abort_flag)) ok = false;
      if (ok) ok = scores(0);
      if (ok && n_tiles > 1) ok = scores(1);
      for (int it = 0; ok && it < n_tiles; ++it) {
        const int st = it & 1;
        if (!wait_bar(&p_ready[st], (it >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!wait_bar(&v_full[st], (it >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {               // 16 keys per instruction: 8 columns of P
          const uint32_t vb = smem_addr(v_s + st * NSUB * KV_SUB_BYTES) + kk * 16 * 128;
          umma_bf16_a_tmem(tmem_base + O_COL, tmem_base + st * BN + kk * 8, smem_desc_mn128(vb, KV_SUB_BYTES), IDESC_O,
                           (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[st]);
        umma_commit(&v_empty[st]);
        if (it + 2 < n_tiles && !scores(it + 2)) { ok = false; break; }
      }
    }
  } else {
    // ---------------- softmax: thread = query row ----------------
    const int r = warp * 32 + lane;
    const int i = i0 + r;                                    // position of this row's query
    const uint32_t lane_bits = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    for (int it = 0; ok && it < n_tiles; ++it) {
      const int st = it & 1, j0 = (kt_lo + it) * BN;
      if (!wait_bar(&s_full[st], (it >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      float sc[BN];
      {
        uint32_t raw[BN];
#pragma unroll
        for (int c = 0; c < BN; c += 16) tmem_ld16_issue(tmem_base + lane_bits + st * BN + c, raw + c);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < BN; ++c) sc[c] = __uint_as_float(raw[c]);
      }
      // Scores stay raw; the scale (> 0) is folded into the exponent: p = 2^(s * scale - m).
      // A tile that every row sees entirely (the common case) takes the path without masks.
      const bool need_mask = (j0 + BN - 1 > i0) || (p.window > 0 && j0 < i0 + BM - 1 - (p.window - 1)) || (j0 + BN > len);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < BN; ++c) {
          const int j = j0 + c;
          const bool vis = j <= i && j < len && (p.window <= 0 || j >= i - (p.window - 1));
          if (!vis) sc[c] = -INFINITY;
        }
      }
      float mx;
      {                                                      // four chains of three-input maxima
        float m4[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const float* s16 = sc + 16 * g;
          float m = max3(s16[0], s16[1], s16[2]);
#pragma unroll
          for (int c = 3; c < 15; c += 2) m = max3(m, s16[c], s16[c + 1]);
          m4[g] = fmaxf(m, s16[15]);
        }
        mx = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]);
      }
      mx *= p.scale_log2e;                                   // -inf stays -inf
      const bool grow = mx > m_used + 8.0f || (m_used == -INFINITY && mx != -INFINITY);
      const bool warp_grow = __any_sync(0xffffffffu, grow);
      if (warp_grow) {
        // the output so far refers to the old maximum: rescale it once the MMAs that add to it are done
        if (it > 0 && !wait_bar(&pv_done[(it - 1) & 1], ((it - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
        const float m_new = grow ? fmaxf(m_used, mx) : m_used;
        const float alpha = !grow ? 1.f : (m_used == -INFINITY ? 0.f : ex2(m_used - m_new));
        m_used = m_new;
        l *= alpha;
        if (it > 0) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < HD; c += 16) {
            float o[16];
            tmem_ld16(tmem_base + lane_bits + O_COL + c, o);
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] *= alpha;
            tmem_st16(tmem_base + lane_bits + O_COL + c, o);
          }
          tc_fence_before();
        }
      }
      // P as bf16 over the first half of this tile's scores in tensor memory (each thread has read its whole
      // row of scores before it writes): two keys per 32-bit column, the lower key in the lower half.
      // Two scores per instruction (packed fp32 FMA and add).  A masked score is -inf and stays -inf through
      // the FMA (the scale is positive, -m finite), and 2^-inf is 0: masked keys need no select here.
      const float neg_m = m_used == -INFINITY ? 0.f : -m_used;   // a row without a visible key: all p are 0
      const uint64_t scale2 = pack2(p.scale_log2e, p.scale_log2e), neg_m2 = pack2(neg_m, neg_m);
      uint64_t l2a = pack2(0.f, 0.f), l2b = l2a;
      uint32_t pk[BN / 2];
#pragma unroll
      for (int c = 0; c < BN / 2; ++c) {
        float ea, eb;
        unpack2(fma2(pack2(sc[2 * c], sc[2 * c + 1]), scale2, neg_m2), ea, eb);
        const float pa = ex2(ea), pb = ex2(eb);
        if (c & 1) l2b = add2(l2b, pack2(pa, pb)); else l2a = add2(l2a, pack2(pa, pb));
        const __nv_bfloat162 two = __floats2bfloat162_rn(pa, pb);
        pk[c] = *reinterpret_cast<const uint32_t*>(&two);
      }
#pragma unroll
      for (int c = 0; c < BN / 2; c += 16) tmem_st16_issue(tmem_base + lane_bits + st * BN + c, pk + c);
      tmem_st_wait();
      float l0, l1;
      unpack2(add2(l2a, l2b), l0, l1);
      l += l0 + l1;
      tc_fence_before();
      mbar_arrive(&p_ready[st]);
    }
    if (ok && !wait_bar(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag)) ok = false;
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((long long)(q_begin + i) * p.heads + head) * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 16) {
        float o[16];
        tmem_ld16(tmem_base + lane_bits + O_COL + c, o);
        if (i < len) {
          uint4 w2[2];
          __nv_bfloat162* wp = reinterpret_cast<__nv_bfloat162*>(w2);
#pragma unroll
          for (int e = 0; e < 8; ++e) wp[e] = __floats2bfloat162_rn(o[2 * e] * inv, o[2 * e + 1] * inv);
          reinterpret_cast<uint4*>(dst + c)[0] = w2[0];
          reinterpret_cast<uint4*>(dst + c)[1] = w2[1];
        }
      }
    }
  }
  if (!ok && lane == 0) {
    if (!*abort_flag) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
    *abort_flag = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

IERT_API int iert_attention_prefill_tc_available() { return 1; }

// Same contract as iert_attention_prefill; additionally qkv must be 16-byte aligned.  Returns
// IERT_BAD_ARGUMENT (nothing launched) when the tensor map cannot be made.
IERT_API int iert_attention_prefill_tc(const void* qkv, void* out, const IertBatchView* batch, int heads,
                                       int kv_heads, int window, float scale, int max_q_len, int* err,
                                       cudaStream_t stream) {
  if (batch->n_tokens <= 0 || max_q_len <= 0) return IERT_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || (max_q_len + BM - 1) / BM > 65535 || batch->n_seqs > 65535 ||
      ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15))
    return IERT_BAD_ARGUMENT;
  const long long width = (long long)(heads + 2 * kv_heads) * HD;
  CUtensorMap map_q, map_kv;
  if (!tma_host::tensor_map_2d(qkv, batch->n_tokens, width, width, BM, &map_q) ||
      !tma_host::tensor_map_2d(qkv, batch->n_tokens, width, width, BN, &map_kv))
    return IERT_BAD_ARGUMENT;
  PrefillTcParams p;
  p.out = (__nv_bfloat16*)out;
  p.heads = heads; p.kv_heads = kv_heads; p.window = window;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.err = err;
  const size_t smem = (size_t)NSUB * SUB_BYTES + 4 * (size_t)NSUB * KV_SUB_BYTES + 256;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return IERT_CUDA_ERROR;
    }
    configured = true;
  }
  dim3 grid(heads, (max_q_len + BM - 1) / BM, batch->n_seqs);
  launch_dep(attention_prefill_tc_kernel, grid, dim3(THREADS), smem, stream, map_q, map_kv, p, *batch);
  return cudaGetLastError() == cudaSuccess ? IERT_OK : IERT_CUDA_ERROR;
}

#else   // other head sizes: the mma.sync kernel serves them

IERT_API int iert_attention_prefill_tc_available() { return 0; }
IERT_API int iert_attention_prefill_tc(const void*, void*, const IertBatchView*, int, int, int, float, int, int*,
                                       cudaStream_t) {
  return IERT_BAD_ARGUMENT;
}

#endif
