// Prompt attention: causal, optional sliding window, grouped heads, for prompts of unequal
// lengths packed back to back; bf16 operands on the tensor cores (mma.sync m16n8k16), fp32
// scores, softmax and accumulation, in one pass over the keys (running maximum and sum).
// Compiled once per head size: -DHEAD_DIM=<multiple of 16, up to 256>.
//
//   grid (query tiles, heads, sequences); a CTA of 8 warps owns 128 consecutive queries of one
//   head of one sequence, each warp 16 of them.  Key/value tiles of 64 positions come from
//   the step's own packed projection (a prompt starts at position 0, so every key it attends
//   to is in the step) through cp.async into double-buffered shared memory whose rows are
//   padded by 16 bytes, which makes every ldmatrix conflict-free for any head size.
//   Visible keys of query i: j in [max(0, i - (W - 1)), i] (src/layers/attention.rs:364-368);
//   tiles entirely outside are never loaded, tiles entirely inside skip the mask.
//
// Formulas: src/layers/attention.rs:357-415, src/ops/softmax.rs:11-25.
#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16>"
#endif

using namespace iert;

namespace {

constexpr int HD = HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");
constexpr int BN = 64, WARPS = 8, BM = WARPS * 16, THREADS = WARPS * 32;
constexpr int ROW_BYTES = HD * 2 + 16;                 // padded row of a tile in shared memory
constexpr int TILE_BYTES = BN * ROW_BYTES;                // a key or value tile
constexpr int Q_TILE_BYTES = BM * ROW_BYTES;
constexpr int KSTEPS = HD / 16;                        // k-steps of Q.K^T; also 16-wide column pairs of the output
constexpr bool Q_IN_REGS = HD <= 128;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;                        // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (fp32 in, fp32 out, about 2 ulp).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copy ROWS x HD bf16 (row stride `ld` elements) into a padded tile; rows >= n_valid become zeros.
template <int ROWS>
__device__ __forceinline__ void load_tile(uint8_t* tile, const __nv_bfloat16* src, long long ld, int n_valid) {
  constexpr int CHUNKS = HD / 8;                       // 16-byte chunks per row
  for (int i = threadIdx.x; i < ROWS * CHUNKS; i += THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const bool ok = r < n_valid;
    cp_async16(tile + r * ROW_BYTES + c * 16, src + (ok ? (long long)r * ld + c * 8 : 0), ok);
  }
}

__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out,
                         IertBatchView b, int heads, int kv_heads, int window, float scale_log2e) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* q_tile = smem;
  auto k_tile = [&](int i) { return smem + Q_TILE_BYTES + i * TILE_BYTES; };
  auto v_tile = [&](int i) { return smem + Q_TILE_BYTES + (2 + i) * TILE_BYTES; };

  const int s = blockIdx.z, head = blockIdx.y;
  if (b.slot_ids[s] < 0) return;
  const int q_begin = b.cu_q[s], len = b.cu_q[s + 1] - q_begin;
  const int n_qt = (len + BM - 1) / BM;
  const int qt = n_qt - 1 - (int)blockIdx.x;            // the longest tiles (latest queries) start first
  if (qt < 0) return;
  const int i0 = qt * BM;
  const int kvh = head / (heads / kv_heads);
  const long long ld = (long long)(heads + 2 * kv_heads) * HD;
  const __nv_bfloat16* q_src = qkv + (long long)(q_begin + i0) * ld + (long long)head * HD;
  const __nv_bfloat16* k_src = qkv + (long long)q_begin * ld + (long long)(heads + kvh) * HD;
  const __nv_bfloat16* v_src = k_src + (long long)kv_heads * HD;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int i_hi = min(len, i0 + BM) - 1;               // last valid query of the tile
  const int j_lo = window > 0 ? max(0, i0 - (window - 1)) : 0;
  const int kt_lo = j_lo / BN, kt_hi = i_hi / BN;       // key tiles to visit, inclusive

  load_tile<BM>(q_tile, q_src, ld, len - i0);
  load_tile<BN>(k_tile(0), k_src + (long long)kt_lo * BN * ld, ld, len - kt_lo * BN);
  load_tile<BN>(v_tile(0), v_src + (long long)kt_lo * BN * ld, ld, len - kt_lo * BN);
  cp_async_commit();

  uint32_t q_frag[Q_IN_REGS ? KSTEPS : 1][4];
  float o[KSTEPS * 2][4];
#pragma unroll
  for (int n = 0; n < KSTEPS * 2; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};   // rows g and g + 8 of the warp's 16
  const int qi[2] = {i0 + warp * 16 + g, i0 + warp * 16 + g + 8};   // their positions in the sequence

  for (int kt = kt_lo; kt <= kt_hi; ++kt) {
    const int buf = (kt - kt_lo) & 1;
    if (kt < kt_hi) {                                   // prefetch the next tile into the other buffer
      load_tile<BN>(k_tile(buf ^ 1), k_src + (long long)(kt + 1) * BN * ld, ld, len - (kt + 1) * BN);
      load_tile<BN>(v_tile(buf ^ 1), v_src + (long long)(kt + 1) * BN * ld, ld, len - (kt + 1) * BN);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if constexpr (Q_IN_REGS) {
      if (kt == kt_lo) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
          ldmatrix_x4(q_frag[ks], q_tile + (warp * 16 + (lane & 15)) * ROW_BYTES + (ks * 16 + (lane >> 4) * 8) * 2);
      }
    }

    // ---- S = Q K^T for this warp's 16 queries and the tile's 64 keys
    float sc[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t qa[4];
      if constexpr (Q_IN_REGS) { qa[0] = q_frag[ks][0]; qa[1] = q_frag[ks][1]; qa[2] = q_frag[ks][2]; qa[3] = q_frag[ks][3]; }
      else ldmatrix_x4(qa, q_tile + (warp * 16 + (lane & 15)) * ROW_BYTES + (ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {            // pairs of 8-key column tiles
        uint32_t kb[4];
        ldmatrix_x4(kb, k_tile(buf) + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * ROW_BYTES +
                            (ks * 16 + ((lane >> 3) & 1) * 8) * 2);
        mma_bf16(sc[2 * np], qa, kb[0], kb[1]);
        mma_bf16(sc[2 * np + 1], qa, kb[2], kb[3]);
      }
    }

    // ---- scale, mask, running softmax (base 2: scale_log2e = scale * log2(e))
    const int j0 = kt * BN;
    const bool need_mask = (j0 + BN - 1 > i0 + warp * 16) || (window > 0 && j0 < i0 + warp * 16 + 15 - (window - 1)) ||
                           (j0 + BN > len);
    float m_new[2] = {m_row[0], m_row[1]};
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = sc[n][e] * scale_log2e;
        if (need_mask) {
          const int j = j0 + n * 8 + tq * 2 + (e & 1), i = qi[e >> 1];
          const bool vis = j <= i && j < len && (window <= 0 || j >= i - (window - 1));
          if (!vis) v = -INFINITY;
        }
        sc[n][e] = v;
        m_new[e >> 1] = fmaxf(m_new[e >> 1], v);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
      m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
      alpha[r] = m_row[r] == -INFINITY ? 0.f : fast_exp2(m_row[r] - m_new[r]);
      m_row[r] = m_new[r];
      l_row[r] *= alpha[r];
    }
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mr = m_new[e >> 1];
        const float pv = (sc[n][e] == -INFINITY || mr == -INFINITY) ? 0.f : fast_exp2(sc[n][e] - mr);
        sc[n][e] = pv;
        l_row[e >> 1] += pv;                            // this thread's share; reduced over the quad at the end
      }
    }
#pragma unroll
    for (int n = 0; n < KSTEPS * 2; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t pa[4] = {pack_bf16(sc[2 * kk][0], sc[2 * kk][1]), pack_bf16(sc[2 * kk][2], sc[2 * kk][3]),
                        pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3])};
#pragma unroll
      for (int dp = 0; dp < KSTEPS; ++dp) {             // pairs of 8-wide output column tiles
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, v_tile(buf) + (kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * ROW_BYTES +
                                  (dp * 16 + (lane >> 4) * 8) * 2);
        mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
        mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();                                    // the buffer is refilled two iterations later
  }

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
    l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (qi[r] >= len) continue;
    const float inv = l_row[r] > 0.f ? 1.0f / l_row[r] : 0.f;
    __nv_bfloat16* dst = out + ((long long)(q_begin + qi[r]) * heads + head) * HD;
#pragma unroll
    for (int n = 0; n < KSTEPS * 2; ++n)
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + tq * 2) =
          __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
  }
}

}  // namespace

IERT_API int iert_attention_prefill_head_dim() { return HD; }

// qkv: packed bf16 [T, (heads + 2 kv_heads) * HEAD_DIM], queries and keys rotated.
// out: bf16 [T, heads * HEAD_DIM].  Every sequence of the step starts at position 0.
// max_q_len: the longest sequence of the step (sizes the grid).
IERT_API int iert_attention_prefill(const void* qkv, void* out, const IertBatchView* batch, int heads,
                                    int kv_heads, int window, float scale, int max_q_len,
                                    cudaStream_t stream) {
  if (batch->n_tokens <= 0 || max_q_len <= 0) return IERT_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || heads > 65535 || batch->n_seqs > 65535)
    return IERT_BAD_ARGUMENT;
  const size_t smem = (size_t)Q_TILE_BYTES + 4 * (size_t)TILE_BYTES;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return IERT_CUDA_ERROR;
    }
    configured = true;
  }
  dim3 grid((max_q_len + BM - 1) / BM, heads, batch->n_seqs);
  attention_prefill_kernel<<<grid, THREADS, smem, stream>>>(
      (const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, *batch, heads, kv_heads, window,
      scale * 1.4426950408889634f);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? IERT_OK : IERT_CUDA_ERROR;
}
