// Projection for one-token steps without split-K: out[t, n] = sum_k x[t, k] * w[n, k] for up to 32
// tokens, bf16 operands, fp32 accumulation.
//
// Why a second projection kernel.  With a handful of tokens a projection is a stream of its weight
// matrix, and the tcgen05 kernel (gemm_tc.cu) can only cut that stream into tiles of 128 weight
// rows: a 4,096-row matrix gives 32 tiles for 148 SMs, so it has to split k over several CTAs and
// add their partial tiles through memory, with a counter and a wait for the slowest split.  That
// epilogue is 5 to 7 us of a 9 to 19 us launch in a decoding step of a 7B model, during which
// nothing streams.  Here a CTA owns 16 weight rows over ALL of k (mma.sync m16n8k16: 16 rows of
// the matrix x 8 tokens), so 4,096 rows are 256 CTAs that never talk to each other: the epilogue
// is one addition of four warps' registers through shared memory and one read-modify-write of the
// residual.  The tensor-core rate of mma.sync is irrelevant at this size; bytes per second count.
//
//   grid   ceil(N / 16) CTAs, 160 threads: four computing warps and one producer warp.
//   ring   a stage holds eight k-blocks of 64 (two per computing warp): per k-block the CTA's 16
//          weight rows (2 KB) and the tokens (8 x NT rows, 1 KB each 8), fetched by TMA with the
//          128-byte swizzle (conflict-free ldmatrix); when k is a multiple of 64 one copy brings a
//          stage's weights and one its tokens (the matrix seen as k-blocks of [rows, 64]), else one
//          copy per k-block.  Weights do not depend on the kernel in
//          front, tokens do: the producer asks for the weights of the first stages before it waits
//          for that kernel (programmatic dependent launch), then for their tokens.
//   warp w multiplies k-blocks 8 s + w and 8 s + w + 4 of every stage s; its accumulators (16 rows x 8 NT tokens)
//          stay in registers to the end; the four warps are added in warp order (a fixed order:
//          results are repeatable to the bit), then stored or added into the fp32 residual.
// Every wait on a barrier is bounded; when one runs out the kernel sets IERT_ERR_WAIT_EXPIRED,
// waits (bounded) for the copies it has asked for, and returns.
#include "common.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

#include <cstring>

using namespace iert;

namespace {

constexpr int ROWS = 16;                  // weight rows per CTA
constexpr int KB = 64;                    // elements per k-block: one 128-byte swizzle row
constexpr int WARPS = 4, THREADS = WARPS * 32 + 32;
constexpr int KPS = 8;                    // k-blocks per ring stage: two per computing warp
constexpr int W_BYTES = ROWS * KB * 2;    // one k-block of the CTA's rows
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr int MAX_STAGES = 16;

enum : int { MODE_STORE = 0, MODE_ADD_RESIDUAL = 1 };

// Built with -DIERT_GEMM_TRACE (IERT_EXTRA_DEFINES=IERT_GEMM_TRACE), the last 64 launches record when
// their CTAs pass six points, on the device-wide nanosecond timer; read with iert_gemm_rows_trace_read.
// A measuring aid: without the definition nothing of it is compiled.
#ifdef IERT_GEMM_TRACE
constexpr int TRACE_LAUNCHES = 64, TRACE_CTAS = 512, TRACE_EVENTS = 8;
__device__ unsigned long long g_rows_trace[TRACE_LAUNCHES][TRACE_CTAS][TRACE_EVENTS];
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define IERT_TRACE(ev)                                                                                         \
  do { if (p.trace_seq >= 0 && blockIdx.x < TRACE_CTAS) g_rows_trace[p.trace_seq][blockIdx.x][ev] = global_ns(); } while (0)
#else
#define IERT_TRACE(ev) do {} while (0)
#endif

struct RowsParams {
  void* out;
  long long ldo;
  int out_dtype, mode;
  int M, N, K;
  int kb_total, n_stages, stages;         // k-blocks, ring uses (KPS k-blocks each), ring depth
  int boxes3d;                            // K is a multiple of 64: one copy brings a stage's weights, one its tokens
  int* err;
  IertRowScale scale;                     // scale.sumsq != null: the outputs are multiplied by the rows' 1 / rms
  IertNormAhead ahead;                    // ahead.scaled_out != null (residual add): the next norm's first half
  int trace_seq;
};

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm2(uint32_t (&r)[2], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// The 16-byte chunk holding elements [col, col + 8) of row `row` of a tile written by TMA with the
// 128-byte swizzle (rows of 128 bytes; the tile starts on a 1,024-byte boundary).
__device__ __forceinline__ const uint8_t* swz(const uint8_t* tile, int row, int col) {
  return tile + row * 128 + ((((col >> 3) ^ (row & 7))) << 4);
}
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (sm100::mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  return false;
}

// NT: groups of 8 tokens (1, 2 or 4).
template <int NT>
__global__ void __launch_bounds__(THREADS)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const RowsParams p) {
  constexpr int X_BYTES = NT * 8 * KB * 2;                 // one k-block of the tokens
  constexpr int X_OFF = KPS * W_BYTES;                     // a stage: its KPS weight tiles, then its KPS token tiles
  constexpr int STAGE_BYTES = KPS * (W_BYTES + X_BYTES);
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[MAX_STAGES], empty[MAX_STAGES];
  __shared__ int abort_s;
  __shared__ float rstd_s[32];
  uint8_t* smem = smem_raw + ((1024u - (sm100::smem_addr(smem_raw) & 1023u)) & 1023u);
  volatile int* abort_flag = &abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int n0 = blockIdx.x * ROWS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { sm100::mbar_init(&full[s], 1); sm100::mbar_init(&empty[s], WARPS); }
    abort_s = 0;
    sm100::mbar_fence_init();
    sm100::tma_prefetch_desc(&map_w);
    sm100::tma_prefetch_desc(&map_x);
  }
  __syncthreads();
  if (threadIdx.x == 0) { pdl_launch_dependents(); IERT_TRACE(0); }

  if (warp == WARPS) {
    // ---------------- producer ----------------
    if (lane == 0) {
      bool ok = true, dep_ready = false;
      int armed = 0;                                        // ring uses asked for so far
      // the weights / the tokens of ring use s into slot st (k-blocks beyond K read as zeros)
      auto load_w = [&](int s, int st) {
        uint8_t* base = smem + (size_t)st * STAGE_BYTES;
        if (p.boxes3d) { sm100::tma_load_3d(base, &map_w, &full[st], 0, n0, s * KPS); return; }
#pragma unroll
        for (int j = 0; j < KPS; ++j) sm100::tma_load_2d(base + j * W_BYTES, &map_w, &full[st], (s * KPS + j) * KB, n0);
      };
      auto load_x = [&](int s, int st) {
        uint8_t* base = smem + (size_t)st * STAGE_BYTES + X_OFF;
        if (p.boxes3d) { sm100::tma_load_3d(base, &map_x, &full[st], 0, 0, s * KPS); return; }
#pragma unroll
        for (int j = 0; j < KPS; ++j) sm100::tma_load_2d(base + j * X_BYTES, &map_x, &full[st], (s * KPS + j) * KB, 0);
      };
      for (int s = 0; s < p.n_stages && ok; ++s) {
        const int st = s % stages;
        if (!dep_ready && s == stages) {
          // the ring is full of weights: now wait for the kernel in front and ask for their tokens
          pdl_wait();
          IERT_TRACE(2);
          for (int i = 0; i < stages; ++i) load_x(i, i);
          dep_ready = true;
        }
        if (s >= stages && !wait_or_abort(&empty[st], ((uint32_t)(s / stages) - 1u) & 1u, abort_flag)) { ok = false; break; }
        sm100::mbar_expect_tx(&full[st], STAGE_BYTES);
        if (s == 0) IERT_TRACE(1);
        if (s == p.n_stages - 1) IERT_TRACE(3);
        load_w(s, st);
        if (dep_ready) load_x(s, st);
        armed = s + 1;
      }
      if (!dep_ready) {
        pdl_wait();
        IERT_TRACE(2);
        for (int i = 0; i < armed; ++i) load_x(i, i);
      }
      if (!ok) {
        if (!*abort_flag) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
        *abort_flag = 1;
        // the copies already asked for land whether or not anyone uses them: wait for the last
        // use asked for in every slot before the CTA leaves
        for (int st = 0; st < stages && st < armed; ++st) {
          const int last = ((armed - 1 - st) / stages) * stages + st;
          sm100::mbar_wait(&full[st], (uint32_t)(last / stages) & 1u, WAIT_LIMIT);
        }
      }
    }
  } else {
    // ---------------- four computing warps ----------------
    if (p.scale.sumsq) {                  // the input rows' 1 / rms, while the first weights are on their way
      pdl_wait();
      row_scales_from_parts(p.scale, p.M, rstd_s, threadIdx.x, WARPS * 32);
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
    bool ok = true;
    for (int s = 0; s < p.n_stages; ++s) {
      const int st = s % stages;
      if (!wait_or_abort(&full[st], (uint32_t)(s / stages) & 1u, abort_flag)) { ok = false; break; }
      if (threadIdx.x == 0 && s == 0) IERT_TRACE(4);
      if (threadIdx.x == 0 && s == p.n_stages - 1) IERT_TRACE(5);
#pragma unroll
      for (int j = 0; j < KPS / WARPS; ++j) {
        const int kbi = warp + j * WARPS;                       // this warp's k-blocks of the stage
        const uint8_t* wt = smem + (size_t)st * STAGE_BYTES + kbi * W_BYTES;
        const uint8_t* xt = smem + (size_t)st * STAGE_BYTES + X_OFF + kbi * X_BYTES;
#pragma unroll
        for (int ks = 0; ks < KB / 16; ++ks) {
          uint32_t a[4];
          ldsm4(a, swz(wt, lane & 15, ks * 16 + (lane >> 4) * 8));
          if constexpr (NT == 1) {
            uint32_t b[2];
            ldsm2(b, swz(xt, lane & 7, ks * 16 + ((lane >> 3) & 1) * 8));
            mma16816(acc[0], a, b[0], b[1]);
          } else {
#pragma unroll
            for (int t2 = 0; t2 < NT / 2; ++t2) {
              uint32_t b[4];
              ldsm4(b, swz(xt, t2 * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 16 + ((lane >> 3) & 1) * 8));
              mma16816(acc[2 * t2], a, b[0], b[1]);
              mma16816(acc[2 * t2 + 1], a, b[2], b[3]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&empty[st]);
    }
    if (!ok && lane == 0) {
      if (!*abort_flag) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
      *abort_flag = 1;
    }
    // ---- the four warps' sums, added in warp order; every stage of the ring has been used
    asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");
    if (*abort_flag) {
      // a wait ran out somewhere in this CTA: before it leaves, wait (bounded) for whatever the
      // producer may still have asked for into the ring
      if (threadIdx.x == 0) {
        for (int st = 0; st < stages && st < p.n_stages; ++st) {
          const int last = ((p.n_stages - 1 - st) / stages) * stages + st;
          sm100::mbar_wait(&full[st], (uint32_t)(last / stages) & 1u, WAIT_LIMIT);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");
    } else {
      pdl_wait();      // (returned long ago for the producer; here for the writes below)
      float* red = reinterpret_cast<float*>(smem);            // [WARPS][ROWS][NT * 8]
      const int g = lane >> 2, tq = lane & 3;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        float* r0 = red + ((size_t)warp * ROWS + g) * (NT * 8) + t * 8 + tq * 2;
        r0[0] = acc[t][0]; r0[1] = acc[t][1];
        r0[8 * NT * 8] = acc[t][2]; r0[8 * NT * 8 + 1] = acc[t][3];        // row g + 8
      }
      asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");
      // thread -> (token, row): consecutive threads walk the 16 rows of one token (64 contiguous bytes of
      // out); the 16 threads of a token are half a warp
      for (int i = threadIdx.x; i < ROWS * NT * 8; i += WARPS * 32) {
        const int tok = i / ROWS, row = i % ROWS, n = n0 + row;
        const bool live = tok < p.M && n < p.N;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[((size_t)w * ROWS + row) * (NT * 8) + tok];
        if (p.scale.sumsq && tok < p.M) v *= rstd_s[tok];
        if (live) {
          if (p.out_dtype == IERT_F32) {
            float* o = (float*)p.out + (long long)tok * p.ldo + n;
            if (p.mode == MODE_ADD_RESIDUAL) v += *o;
            *o = v;
          } else {
            ((__nv_bfloat16*)p.out)[(long long)tok * p.ldo + n] = __float2bfloat16_rn(v);
          }
        }
        if (p.ahead.scaled_out) {           // (the same for every thread) v is the new residual value
          float ss = 0.f;
          if (live) {
            const float g = p.ahead.weight_dtype == IERT_F32 ? ((const float*)p.ahead.weight)[n]
                                                             : __bfloat162float(((const __nv_bfloat16*)p.ahead.weight)[n]);
            ((__nv_bfloat16*)p.ahead.scaled_out)[(long long)tok * p.ahead.ld + n] = __float2bfloat16_rn(v * g);
            ss = v * v;
          }
          ss += __shfl_xor_sync(0xffffffffu, ss, 8);
          ss += __shfl_xor_sync(0xffffffffu, ss, 4);
          ss += __shfl_xor_sync(0xffffffffu, ss, 2);
          ss += __shfl_xor_sync(0xffffffffu, ss, 1);
          if (row == 0 && tok < p.M) p.ahead.sumsq_out[(size_t)tok * p.ahead.parts + blockIdx.x] = ss;
        }
      }
    }
    if (threadIdx.x == 0) IERT_TRACE(7);
  }
}

#ifdef IERT_GEMM_TRACE
int g_trace_meta[TRACE_LAUNCHES][8];
int g_trace_next = 0;
#endif

template <int NT>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const RowsParams& p, int grid, cudaStream_t stream) {
  constexpr int STAGE_BYTES = KPS * (W_BYTES + NT * 8 * KB * 2);
  const size_t smem = (size_t)p.stages * STAGE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_rows_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess)
      return iert_check_launch("gemm_rows attribute");
    configured = true;
  }
  RowsParams q = p;
  q.trace_seq = -1;
#ifdef IERT_GEMM_TRACE
  q.trace_seq = g_trace_next % TRACE_LAUNCHES;
  int* tm = g_trace_meta[q.trace_seq];
  tm[0] = g_trace_next++; tm[1] = p.M; tm[2] = p.N; tm[3] = p.K; tm[4] = grid; tm[5] = NT; tm[6] = p.stages; tm[7] = p.mode;
#endif
  launch_dep(gemm_rows_kernel<NT>, dim3(grid), dim3(THREADS), smem, stream, mw, mx, q);
  return iert_check_launch("gemm_rows");
}

}  // namespace

#ifdef IERT_GEMM_TRACE
// stamps: [64][512][8] unsigned 64-bit; meta: [64][8] int (sequence number, M, N, K, grid, token groups, stages, mode)
IERT_API int iert_gemm_rows_trace_read(unsigned long long* stamps, int* meta) {
  if (cudaMemcpyFromSymbol(stamps, g_rows_trace, sizeof(unsigned long long) * TRACE_LAUNCHES * TRACE_CTAS * TRACE_EVENTS) != cudaSuccess)
    return IERT_CUDA_ERROR;
  memcpy(meta, g_trace_meta, sizeof(g_trace_meta));
  return IERT_OK;
}
#endif

// x: [M, K] bf16 (M <= 32), row stride ldx; w: [N, K] bf16, row stride ldw; out: [M, N] of out_dtype,
// row stride ldo.  mode 0 stores, mode 1 adds into out (fp32).  K, ldx and ldw must be multiples of
// 8 and the pointers 16-byte aligned (TMA); otherwise, or with more than 32 tokens,
// IERT_BAD_ARGUMENT is returned and nothing is launched.  force_stages: 0 = choose.
//   scale (optional)  the rows of x are the first half of an RMSNorm (IertNormAhead of the kernel that
//                     wrote them): the outputs are multiplied by each row's 1 / rms (see common.cuh).
//   ahead (optional; mode 1)  the first half of the NEXT norm over the new rows of `out`: ahead->parts
//                     is set to the number of partial sums per row written (one per CTA).
IERT_API int iert_gemm_rows(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype,
                            long long ldo, int M, int N, int K, int mode, const IertRowScale* scale,
                            IertNormAhead* ahead, int force_stages, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IERT_OK;
  if (M > 32 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return IERT_BAD_ARGUMENT;
  if (mode != MODE_STORE && mode != MODE_ADD_RESIDUAL) return IERT_BAD_ARGUMENT;
  if (out_dtype != IERT_F32 && out_dtype != IERT_BF16) return IERT_BAD_ARGUMENT;
  if (mode == MODE_ADD_RESIDUAL && out_dtype != IERT_F32) return IERT_BAD_ARGUMENT;
  if (scale && (!scale->sumsq || scale->parts <= 0 || scale->hidden <= 0)) return IERT_BAD_ARGUMENT;
  if (ahead && (mode != MODE_ADD_RESIDUAL || !ahead->weight || !ahead->scaled_out || !ahead->sumsq_out ||
                (ahead->weight_dtype != IERT_F32 && ahead->weight_dtype != IERT_BF16)))
    return IERT_BAD_ARGUMENT;
  const int nt = M <= 8 ? 1 : M <= 16 ? 2 : 4;
  RowsParams p;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.mode = mode;
  p.M = M; p.N = N; p.K = K; p.err = err;
  p.scale = IertRowScale{nullptr, 0, 0, 0.f};
  if (scale) p.scale = *scale;
  p.ahead = IertNormAhead{nullptr, 0, nullptr, 0, nullptr, 0};
  p.kb_total = (K + KB - 1) / KB;
  p.n_stages = (p.kb_total + KPS - 1) / KPS;
  const int stage_bytes = KPS * (W_BYTES + nt * 8 * KB * 2);
  // The ring is as deep as the SM's shared memory allows for the CTAs that share it: what counts is
  // the bytes in flight per SM (about 200 KB keep the memory system busy), so 256 CTAs on 148 SMs
  // get half an SM each, 384 CTAs a third.
  const int grid = (N + ROWS - 1) / ROWS;
  int sms = iert_sm_count_cached();
  int per_sm = (grid + sms - 1) / sms;
  if (per_sm > 4) per_sm = 4;
  int stages = force_stages ? force_stages : ((224 * 1024) / per_sm - 2048) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages > p.n_stages) stages = p.n_stages;
  if (stages < 1 || (size_t)stages * stage_bytes + 1024 > 226 * 1024) return IERT_BAD_ARGUMENT;
  // the warps' sums are added through the ring's memory
  if ((size_t)stages * stage_bytes < (size_t)WARPS * ROWS * nt * 8 * sizeof(float)) return IERT_BAD_ARGUMENT;
  p.stages = stages;
  CUtensorMap mw, mx;
  p.boxes3d = K % KB == 0 && tma_host::tensor_map_kblocks(w, N, K, ldw, ROWS, KPS, &mw) &&
              tma_host::tensor_map_kblocks(x, M, K, ldx, nt * 8, KPS, &mx);
  if (!p.boxes3d && (!tma_host::tensor_map_2d(w, N, K, ldw, ROWS, &mw) || !tma_host::tensor_map_2d(x, M, K, ldx, nt * 8, &mx)))
    return IERT_BAD_ARGUMENT;
  if (ahead) {
    ahead->parts = grid;
    p.ahead = *ahead;
  }
  switch (nt) {
    case 1: return launch<1>(mw, mx, p, grid, stream);
    case 2: return launch<2>(mw, mx, p, grid, stream);
    default: return launch<4>(mw, mx, p, grid, stream);
  }
}
