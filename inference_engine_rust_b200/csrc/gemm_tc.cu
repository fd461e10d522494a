// Tensor-core projection for sm_100a: out[t, n] = sum_k x[t, k] * w[n, k] with bf16 operands
// and fp32 accumulation, on tcgen05.mma with the accumulator in tensor memory and both
// operands brought into shared memory by TMA (128-byte swizzle).
//
// The weight matrix sits on the MMA's M side (128 weight rows per tile) and the tokens on its
// N side (16..256 per tile), so one kernel serves a prompt of thousands of tokens and a
// decoding step of a few: with few tokens the tile is a thin slab of the weight matrix and
// the kernel is a stream of TMA loads at memory bandwidth.  Persistent CTAs walk a list of
// (tile, k-split) work items.  Warp 0 issues the TMA loads, warp 1 issues the MMAs, warps
// 2-5 read the accumulator back (each its quarter of the TMEM lanes) and write the result;
// two accumulators in TMEM let the read-back of one tile overlap the MMAs of the next.
//
// Split-K (few tokens, few tiles): each split writes its fp32 partial tile to scratch memory
// and counts itself in on the tile's counter.  The partials are added in split order (a fixed
// order: the result does not depend on which CTA finishes when).  Who adds them:
//   * every split its own share of the tile's token rows, once the counter shows that all
//     partials are written, when the whole grid is resident at once (one work item per CTA and
//     no more CTAs than the device holds, checked against the occupancy the driver reports):
//     the addition is then spread over `splits` CTAs.  The wait for the counter is bounded
//     like every other wait here;
//   * otherwise the CTA that counts in last, alone, and no CTA waits for another.
//
// Token-major variant (GATED = true), used for prompts.  Gated: the weight matrix is [gate; up] stacked by rows, a tile holds
// 128 gate rows and the 128 up rows that belong to them as ONE 256-row operand on the MMA's N
// side with 128 tokens on its M side (the full-rate 128 x 256 x 16 instruction), and the
// epilogue (one token per thread) writes silu(gate) * up: the feed-forward's activation never goes
// to memory unfused.  The same kernel with 256 consecutive weight rows per tile is the plain
// prompt projection (store or add into the residual): a thread then owns one token's 16
// consecutive outputs per chunk, so its loads and stores are 16-byte vectors.  Whole tiles only.
//
// Residual adds over many tokens (tiles of 128 or 256 tokens) do not read the residual back:
// the epilogue stages 32 tokens x 128 outputs of its accumulator in shared memory and a TMA
// reduce (cp.reduce.async.bulk.tensor, fp32 add at the destination) adds them in.  When such a
// product's tiles leave the last wave part empty and k is long, the tiles of that wave are cut
// into parts of k whose products are added one after the other in a fixed order (see WorkIter).
//
// Every wait on an mbarrier is bounded; when one runs out the kernel sets
// IERT_ERR_WAIT_EXPIRED in the error word, drains its own TMA copies, frees its TMEM and
// returns.
#include "common.cuh"
#include "sm100.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

using namespace iert;
using namespace sm100;

namespace {

constexpr int TILE_N = 128;        // weight rows per tile (UMMA M)
constexpr int TILE_K = 64;         // bf16 elements per k-block: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int W_STAGE_BYTES = TILE_N * TILE_K * 2;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr int OUT_STAGE_BYTES = 32 * TILE_N * 4;   // residual add by TMA: 32 tokens x 128 outputs fp32, two of them
constexpr int XCH_BYTES = 16 * 64 * 4 + 16 + 256;   // weight-major gated tile: 16 tokens x 64 up values, aligned; 64 row scales

enum : int { MODE_STORE = 0, MODE_ADD_RESIDUAL = 1, MODE_GATED_SILU = 2 };

struct GemmParams {
  void* out;
  long long ldo;
  int out_dtype;
  int mode;
  int M, N, K;        // gated: N = rows of the gate half = columns of the output
  int n_step;         // output columns a tile covers (token-major: 128 gated, 256 plain)
  int second_rows;    // token-major: row of the second 128-row weight box, relative to the tile's first
  int t_tiles, n_tiles, splits, kb_total, kb_per_split, stages;
  float* ws;          // [tiles][splits][BT][TILE_N] fp32 partials (splits > 1)
  int* counters;      // [tiles] tickets, zero between launches
  int coop_reduce;    // splits > 1: every split adds its share of the rows (the grid is co-resident)
  int t_group;        // token tiles per group in the order of the tiles (see tile_coords); t_tiles = one group
  int tma_out;        // residual add through TMA reduce (map_o), weight-major tiles of >= 128 tokens
  int tail_parts;     // > 1: the tiles from full_tiles on are cut into this many parts of k (see WorkIter)
  int full_tiles;
  int* err;
  IertRowScale scale;   // weight-major tiles of up to 64 tokens: scale.sumsq != null: x is the first half of an RMSNorm
                        // (see common.cuh); the outputs (gated: gate and up, before the activation) are multiplied by
                        // the rows' 1 / rms
  IertNormAhead ahead;  // split-K residual add, tiles of 32 or 64 tokens: ahead.scaled_out != null: the reduction also
                        // writes the next norm's first half
  int trace_seq;        // >= 0: the launch's row in the trace (builds with IERT_GEMM_TRACE only)
  uint32_t poll_limit;  // polls of a tile's counter before a CTA gives up waiting for the other CTAs of its tile
};

// Built with -DIERT_GEMM_TRACE (IERT_EXTRA_DEFINES=IERT_GEMM_TRACE), the last 64 launches record when their
// CTAs pass eight points, on the device-wide nanosecond timer; read with iert_gemm_tc_trace_read.  A measuring
// aid: without the definition nothing of it is compiled.
#ifdef IERT_GEMM_TRACE
constexpr int TRACE_LAUNCHES = 64, TRACE_CTAS = 304, TRACE_EVENTS = 8;
__device__ unsigned long long g_tc_trace[TRACE_LAUNCHES][TRACE_CTAS][TRACE_EVENTS];
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define IERT_TRACE(ev)                                                                                       \
  do { if (p.trace_seq >= 0 && blockIdx.x < TRACE_CTAS) g_tc_trace[p.trace_seq][blockIdx.x][ev] = global_ns(); } while (0)
#else
#define IERT_TRACE(ev) do {} while (0)
#endif

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  return false;
}

template <typename TO>
__device__ __forceinline__ void write_out(const GemmParams& p, int tok, int n, float v) {
  TO* o = (TO*)p.out + (long long)tok * p.ldo + n;
  if (p.mode == MODE_ADD_RESIDUAL) *o = from_f32<TO>(to_f32(*o) + v);
  else *o = from_f32<TO>(v);
}
__device__ __forceinline__ void write_out_any(const GemmParams& p, int tok, int n, float v) {
  if (p.out_dtype == IERT_F32) write_out<float>(p, tok, n, v);
  else write_out<__nv_bfloat16>(p, tok, n, v);
}

// Four consecutive outputs of one token, vectorised when aligned and inside the matrix.
__device__ __forceinline__ void write_out4(const GemmParams& p, int tok, int n, const float4& r) {
  const bool whole = n + 4 <= p.N && (p.ldo & 3) == 0 && ((uintptr_t)p.out & 15) == 0;
  if (whole && p.out_dtype == IERT_F32) {
    float4* o = reinterpret_cast<float4*>((float*)p.out + (long long)tok * p.ldo + n);
    if (p.mode == MODE_ADD_RESIDUAL) {
      const float4 a = *o;
      *o = make_float4(a.x + r.x, a.y + r.y, a.z + r.z, a.w + r.w);
    } else {
      *o = r;
    }
  } else if (whole && p.mode == MODE_STORE) {
    uint2 w2;
    *reinterpret_cast<__nv_bfloat162*>(&w2.x) = __floats2bfloat162_rn(r.x, r.y);
    *reinterpret_cast<__nv_bfloat162*>(&w2.y) = __floats2bfloat162_rn(r.z, r.w);
    *reinterpret_cast<uint2*>((__nv_bfloat16*)p.out + (long long)tok * p.ldo + n) = w2;
  } else {
    const float v[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (n + i < p.N) write_out_any(p, tok, n + i, v[i]);
  }
}

// silu(g) * u = g * u / (1 + e^-g).  One exponential and one reciprocal per element (for very
// negative g the exponential overflows to +inf and the quotient is 0, which is the limit).
__device__ __forceinline__ float silu_mul(float g, float u) {
  return __fdividef(g * u, 1.0f + __expf(-g));
}

// Split-K: rows t_first, t_first + 4, ... < t_end of a tile's partial products (one [BT][TILE_N]
// fp32 block per split at `base`) added in split order and written out; 32 threads share a row, each
// four columns (c4).  Four rows and four splits are in flight per thread and pass, and a residual is
// read together with the first partials, so that a pass costs one round trip to the L2: with 64
// rows per split a row-at-a-time loop spent 30 us here.
template <int BT>
__device__ __forceinline__ void reduce_partial_rows(const GemmParams& p, const float* base, int t_first, int t_end,
                                                    int t0, int n, int c4, int n_idx, const float* rstd) {
  const bool vec_res = p.mode == MODE_ADD_RESIDUAL && p.out_dtype == IERT_F32 && n + 4 <= p.N && (p.ldo & 3) == 0 &&
                       ((uintptr_t)p.out & 15) == 0;
  const bool ahead = p.ahead.scaled_out != nullptr;      // (residual add into fp32: checked by the host)
  float g[4] = {0.f, 0.f, 0.f, 0.f};                     // the next norm's scale for this thread's four columns
  if (ahead) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (n + i < p.N)
        g[i] = p.ahead.weight_dtype == IERT_F32 ? ((const float*)p.ahead.weight)[n + i]
                                                : __bfloat162float(((const __nv_bfloat16*)p.ahead.weight)[n + i]);
  }
  for (int t = t_first; t < t_end; t += 16) {
    float4 acc[4], res[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
      res[h] = (vec_res && t + 4 * h < t_end)
                   ? *reinterpret_cast<const float4*>((const float*)p.out + (long long)(t0 + t + 4 * h) * p.ldo + n)
                   : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int s0 = 0; s0 < p.splits; s0 += 4) {
      float4 v[4][4];
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int u = 0; u < 4; ++u)
          v[h][u] = (s0 + u < p.splits && t + 4 * h < t_end)
                        ? __ldcg(reinterpret_cast<const float4*>(base + ((size_t)(s0 + u) * BT + t + 4 * h) * TILE_N) + c4)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          acc[h].x += v[h][u].x; acc[h].y += v[h][u].y; acc[h].z += v[h][u].z; acc[h].w += v[h][u].w;
        }
    }
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      if (t + 4 * h >= t_end) break;                     // the same for the 32 threads that share the row
      const int row = t + 4 * h;
      if (rstd) {                                        // the input rows' 1 / rms (see IertRowScale)
        const float r = rstd[row];
        acc[h].x *= r; acc[h].y *= r; acc[h].z *= r; acc[h].w *= r;
      }
      if (vec_res && !ahead) {
        *reinterpret_cast<float4*>((float*)p.out + (long long)(t0 + row) * p.ldo + n) =
            make_float4(res[h].x + acc[h].x, res[h].y + acc[h].y, res[h].z + acc[h].z, res[h].w + acc[h].w);
      } else if (ahead) {
        // the new residual values, and beside them the next norm's first half (see IertNormAhead)
        float* orow = (float*)p.out + (long long)(t0 + row) * p.ldo;
        float nv[4] = {acc[h].x, acc[h].y, acc[h].z, acc[h].w};
        if (vec_res) {
          nv[0] += res[h].x; nv[1] += res[h].y; nv[2] += res[h].z; nv[3] += res[h].w;
          *reinterpret_cast<float4*>(orow + n) = make_float4(nv[0], nv[1], nv[2], nv[3]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (n + i < p.N) { nv[i] += orow[n + i]; orow[n + i] = nv[i]; } else nv[i] = 0.f;
          }
        }
        __nv_bfloat16* srow = (__nv_bfloat16*)p.ahead.scaled_out + (long long)(t0 + row) * p.ahead.ld;
        if (n + 4 <= p.N && (p.ahead.ld & 3) == 0 && ((uintptr_t)p.ahead.scaled_out & 7) == 0) {
          uint2 w2;
          *reinterpret_cast<__nv_bfloat162*>(&w2.x) = __floats2bfloat162_rn(nv[0] * g[0], nv[1] * g[1]);
          *reinterpret_cast<__nv_bfloat162*>(&w2.y) = __floats2bfloat162_rn(nv[2] * g[2], nv[3] * g[3]);
          *reinterpret_cast<uint2*>(srow + n) = w2;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (n + i < p.N) srow[n + i] = __float2bfloat16_rn(nv[i] * g[i]);
        }
        const float ss = warp_sum(nv[0] * nv[0] + nv[1] * nv[1] + nv[2] * nv[2] + nv[3] * nv[3]);
        if (c4 == 0) p.ahead.sumsq_out[(size_t)(t0 + row) * p.ahead.parts + n_idx] = ss;
      } else {
        write_out4(p, t0 + row, n, acc[h]);
      }
    }
  }
}

// A CTA's list of work, the same for its three roles: items (tile, part of k) strided over the
// grid.  Usually every tile has the same number of parts (p.splits, split-K).  For residual adds
// over many tokens whose tiles leave the last wave part empty (p.tail_parts > 1, one CTA per SM,
// all resident) the first p.full_tiles tiles are whole and each of the others is cut into
// p.tail_parts equal parts of k, listed part by part (all first parts, then all second parts,
// ...), so that the last wave's work comes in pieces a quarter (say) of a tile long and fills
// the SMs evenly, while CTAs that run at the same time still read the same range of k.  The
// parts of a tile add their products into the residual one after the other, in the order of the
// parts, each waiting (bounded) until the tile's counter shows its turn: the order of the
// additions is fixed, the result repeatable, and no scratch memory is used.
// Tile index -> (weight-row tile, token tile).  The token tiles are walked in groups of
// p.t_group: within a group the token tile runs fastest, then the weight-row tile, then the next
// group.  CTAs that run at the same time work on neighbouring tiles and move through k
// together, so a group's activations (sized by the host to stay in the L2) are read from memory
// once and the weight matrix once per group.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& n_idx, int& t_idx) {
  const int tg = min(p.t_group, p.t_tiles);             // any larger value means one group
  const int per_group = tg * p.n_tiles;
  const int group = tile / per_group, r = tile - group * per_group;
  const int in_group = min(tg, p.t_tiles - group * tg);
  n_idx = r / in_group;
  t_idx = group * tg + (r - n_idx * in_group);
}

struct WorkIter {
  const GemmParams& p;
  int work, total_work, n_tail;
  __device__ WorkIter(const GemmParams& p_) : p(p_) {
    const int tiles = p.n_tiles * p.t_tiles;
    n_tail = p.tail_parts > 1 ? tiles - p.full_tiles : 0;
    total_work = p.tail_parts > 1 ? p.full_tiles + n_tail * p.tail_parts : tiles * p.splits;
    work = blockIdx.x;
  }
  // part / n_parts: which part of the tile's k range, out of how many
  __device__ bool next(int& tile, int& part, int& n_parts, int& kb0, int& kb1) {
    if (work >= total_work) return false;
    if (p.tail_parts > 1) {
      if (work < p.full_tiles) {
        tile = work; part = 0; n_parts = 1; kb0 = 0; kb1 = p.kb_total;
      } else {
        const int r = work - p.full_tiles;
        part = r / n_tail; tile = p.full_tiles + r % n_tail; n_parts = p.tail_parts;
        const int per = (p.kb_total + n_parts - 1) / n_parts;
        kb0 = part * per; kb1 = min(p.kb_total, kb0 + per);
      }
    } else {
      part = work % p.splits; tile = work / p.splits; n_parts = p.splits;
      kb0 = part * p.kb_per_split; kb1 = min(p.kb_total, kb0 + p.kb_per_split);
    }
    work += gridDim.x;
    return true;
  }
};

template <int BT, bool GATED>
__global__ void __launch_bounds__(THREADS, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_o, const GemmParams p) {
  constexpr int NW = GATED ? 2 : 1;                             // weight tiles per stage
  constexpr int X_OFF = NW * W_STAGE_BYTES;
  constexpr int STAGE_BYTES = X_OFF + BT * TILE_K * 2;
  constexpr int ACC_STRIDE = NW * BT;                           // TMEM columns of one accumulator stage
  static_assert(2 * ACC_STRIDE <= 512, "two accumulator stages must fit tensor memory");
  constexpr uint32_t ACC_COLS = 2 * ACC_STRIDE < 32 ? 32 : 2 * ACC_STRIDE;   // power of two >= 32
  // plain: 128 weight rows x BT tokens; gated: BT (= 128) tokens x 256 stacked weight rows
  constexpr uint32_t IDESC = GATED ? instr_desc_bf16(BT, 2 * TILE_N) : instr_desc_bf16(TILE_N, BT);
  static_assert(!GATED || BT == 128, "the gated kernel puts 128 tokens on the MMA's M side");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = p.stages;
  uint64_t* full = (uint64_t*)(smem + (size_t)stages * STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* acc_full = empty + stages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* ticket_s = (int*)(tmem_slot + 2);
  uint8_t* xch_s = (uint8_t*)(((uintptr_t)(tmem_slot + 4) + 15) & ~(uintptr_t)15);   // 4 KB, weight-major gated only
  uint8_t* out_s = (uint8_t*)(((uintptr_t)(tmem_slot + 4) + 127) & ~(uintptr_t)127);  // 2 x 16 KB, residual add by TMA only

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  if (warp == 1) tmem_alloc(tmem_slot, ACC_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();
  if (threadIdx.x == 0) IERT_TRACE(0);                       // start

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      // The weight tiles do not depend on the kernel before this one, the token tiles do:
      // the first `stages` weight loads are issued at once, then the dependency is awaited,
      // then their token tiles follow.  (With an ordinary launch the wait returns at once.)
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true, dep_ready = false;
      int pend_kb[12], pend_t0[12];
      WorkIter it(p);
      int tile, split, n_parts, kb0, kb1;
      while (ok && it.next(tile, split, n_parts, kb0, kb1)) {
        int n_idx, t_idx;
        tile_coords(p, tile, n_idx, t_idx);
        const int n0 = n_idx * p.n_step, t0 = t_idx * BT;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!dep_ready && issued == stages) {
            pdl_wait();
            IERT_TRACE(2);                                     // the kernel in front has finished
            for (int i = 0; i < issued; ++i)
              tma_load_2d(smem + (size_t)i * STAGE_BYTES + X_OFF, &map_x, &full[i], pend_kb[i] * TILE_K, pend_t0[i]);
            dep_ready = true;
          }
          if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* ws_ = smem + (size_t)stage * STAGE_BYTES;
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          tma_load_2d(ws_, &map_w, &full[stage], kb * TILE_K, n0);
          if (GATED)   // the second 128 weight rows of the tile: the up rows (gated) or the next rows (plain)
            tma_load_2d(ws_ + W_STAGE_BYTES, &map_w, &full[stage], kb * TILE_K, n0 + p.second_rows);
          else if (p.mode == MODE_GATED_SILU)   // weight-major gated: 64 gate rows (above), then their 64 up rows
            tma_load_2d(ws_ + W_STAGE_BYTES / 2, &map_w, &full[stage], kb * TILE_K, n0 + p.second_rows);
          if (dep_ready) tma_load_2d(ws_ + X_OFF, &map_x, &full[stage], kb * TILE_K, t0);
          else { pend_kb[issued] = kb; pend_t0[issued] = t0; }
          if (issued == 0) IERT_TRACE(1);                    // first weights asked for
          ++issued;
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!dep_ready) {
        pdl_wait();
        IERT_TRACE(2);
        for (int i = 0; i < issued; ++i)
          tma_load_2d(smem + (size_t)i * STAGE_BYTES + X_OFF, &map_x, &full[i], pend_kb[i] * TILE_K, pend_t0[i]);
      }
      if (!ok) {
        if (!*abort_flag) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
        *abort_flag = 1;
        // drain: the copies already issued land whether or not anyone consumes them
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < min(issued, stages); ++i) {
          if (s == 0) { s = stages; ph ^= 1; }
          --s;
          mbar_wait(&full[s], ph, WAIT_LIMIT);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      WorkIter it(p);
      int tile, split, n_parts, kb0, kb1;
      while (ok && it.next(tile, split, n_parts, kb0, kb1)) {
        if (!wait_or_abort(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * ACC_STRIDE);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&full[stage], phase, abort_flag)) { ok = false; break; }
          if (kb == kb0) IERT_TRACE(3);                        // first operands of the (last) work item have arrived
          tc_fence_after();
          const uint32_t w_addr = smem_addr(smem + (size_t)stage * STAGE_BYTES);
          const uint64_t da = smem_desc_k128(w_addr), db = smem_desc_k128(w_addr + X_OFF);
#pragma unroll
          for (int ks = 0; ks < TILE_K / UMMA_K; ++ks) { // 32 bytes further along K per step
            if (GATED)   // tokens on the M side, the 256 stacked weight rows (gate, up) on the N side
              umma_bf16(d_tmem, db + 2 * ks, da + 2 * ks, IDESC, (kb > kb0 || ks > 0) ? 1u : 0u);
            else
              umma_bf16(d_tmem, da + 2 * ks, db + 2 * ks, IDESC, (kb > kb0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        IERT_TRACE(4);                                         // last MMA of the work item issued
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      if (!ok) {
        if (!*abort_flag) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
        *abort_flag = 1;
      }
    }
  } else {
    // ---------------- epilogue: 4 warps, warp w reads TMEM lanes 32*(w%4).. ----------------
    pdl_wait();
    // [64] row scales: behind the gated tile's exchange buffer, or in its place for a plain launch
    float* rstd_s = reinterpret_cast<float*>(p.mode == MODE_GATED_SILU ? xch_s + 16 * 64 * 4 : xch_s);
    const bool scaled = !GATED && BT <= 64 && p.scale.sumsq != nullptr;
    if (scaled) {                          // the rows' 1 / rms, while the weights stream
      row_scales_from_parts(p.scale, p.M < BT ? p.M : BT, rstd_s, (int)threadIdx.x - 64, 128);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    WorkIter it(p);
    int tile, split, n_parts, kb0, kb1;
    while (ok && it.next(tile, split, n_parts, kb0, kb1)) {
      int n_idx, t_idx;
      tile_coords(p, tile, n_idx, t_idx);
      const int n0 = n_idx * p.n_step, t0 = t_idx * BT;
      const int n = n0 + n_local;
      const int t_valid = min(BT, p.M - t0);
      if (!wait_or_abort(&acc_full[acc], acc_phase, abort_flag)) { ok = false; break; }
      if (threadIdx.x == 64) IERT_TRACE(5);                    // the accumulator is complete
      tc_fence_after();
      const bool chained = p.tail_parts > 1 && n_parts > 1;   // a part of a cut tile: adds in its turn
      if (chained && split > 0) {
        if (threadIdx.x == 64) {
          int seen = 0;
          for (uint32_t i = 0; i < p.poll_limit; ++i) {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.counters + tile) : "memory");
            if (seen >= split) break;
            __nanosleep(64);
          }
          if (seen < split) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * ACC_STRIDE);
      float* part = (p.splits > 1 && p.tail_parts <= 1) ? p.ws + ((size_t)(tile * p.splits + split) * BT) * TILE_N + n_local : nullptr;
      if (GATED && p.mode == MODE_GATED_SILU) {
        // lane = token, columns [0, 128) = gate rows, [128, 256) = their up rows
        const int tok = t0 + n_local;
#pragma unroll 1
        for (int c = 0; c < TILE_N; c += 16) {
          float v[16], u[16];
          tmem_ld16(taddr + c, v);
          tmem_ld16(taddr + TILE_N + c, u);
          if (tok < p.M) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (long long)tok * p.ldo + n0 + c;
            if (n0 + c + 16 <= p.N && (p.ldo & 7) == 0 && ((uintptr_t)p.out & 15) == 0) {
              uint4 w2[2];
              __nv_bfloat162* wp = reinterpret_cast<__nv_bfloat162*>(w2);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                wp[j] = __floats2bfloat162_rn(silu_mul(v[2 * j], u[2 * j]), silu_mul(v[2 * j + 1], u[2 * j + 1]));
              reinterpret_cast<uint4*>(o)[0] = w2[0];
              reinterpret_cast<uint4*>(o)[1] = w2[1];
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (n0 + c + j < p.N) o[j] = __float2bfloat16_rn(silu_mul(v[j], u[j]));
            }
          }
        }
      } else if (GATED) {
        // token-major plain product: lane = token, 256 output columns per tile; a thread's 16
        // values of a chunk are contiguous in memory (vector loads and stores)
        const int tok = t0 + n_local;
#pragma unroll 1
        for (int c = 0; c < 2 * TILE_N; c += 16) {
          if (n0 + c >= p.N) break;                    // warp-uniform
          float v[16];
          tmem_ld16(taddr + c, v);
          if (tok >= p.M) continue;
          const bool full16 = n0 + c + 16 <= p.N;
          if (p.out_dtype == IERT_F32) {
            float* o = (float*)p.out + (long long)tok * p.ldo + n0 + c;
            if (full16 && (p.ldo & 3) == 0 && ((uintptr_t)p.out & 15) == 0) {
              float4* o4 = reinterpret_cast<float4*>(o);
              if (p.mode == MODE_ADD_RESIDUAL) {
                float4 r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) r[j] = o4[j];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  o4[j] = make_float4(r[j].x + v[4 * j], r[j].y + v[4 * j + 1], r[j].z + v[4 * j + 2], r[j].w + v[4 * j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) o4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (n0 + c + j < p.N) o[j] = p.mode == MODE_ADD_RESIDUAL ? o[j] + v[j] : v[j];
            }
          } else {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (long long)tok * p.ldo + n0 + c;
            if (full16 && (p.ldo & 7) == 0 && ((uintptr_t)p.out & 15) == 0) {
              uint4 w2[2];
              __nv_bfloat162* wp = reinterpret_cast<__nv_bfloat162*>(w2);
#pragma unroll
              for (int j = 0; j < 8; ++j) wp[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              reinterpret_cast<uint4*>(o)[0] = w2[0];
              reinterpret_cast<uint4*>(o)[1] = w2[1];
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (n0 + c + j < p.N) o[j] = __float2bfloat16_rn(v[j]);
            }
          }
        }
      }
      if (!GATED && p.mode == MODE_GATED_SILU) {
        // Weight-major gated tile: TMEM lanes 0-63 hold 64 gate rows, lanes 64-127 the up rows
        // that belong to them.  The up warps hand their values over through shared memory, the
        // gate warps write silu(gate) * up, 64 consecutive outputs of a token per pair of warps.
        float* xch = reinterpret_cast<float*>(xch_s);                 // [16 tokens][64]
#pragma unroll 1
        for (int c = 0; c < BT; c += 16) {
          if (c >= t_valid) break;                   // uniform over the four warps
          float v[16];
          tmem_ld16(taddr + c, v);
          if (q >= 2) {
#pragma unroll
            for (int j = 0; j < 16; ++j) xch[j * 64 + (n_local - 64)] = v[j];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (q < 2) {
            const int i = n0 + n_local;              // n0 counts gate rows here (64 per tile)
            if (i < p.N) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c + j < t_valid) {
                  const float r = scaled ? rstd_s[c + j] : 1.0f;
                  ((__nv_bfloat16*)p.out)[(long long)(t0 + c + j) * p.ldo + i] =
                      __float2bfloat16_rn(silu_mul(v[j] * r, xch[j * 64 + n_local] * r));
                }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
      // Many tokens, residual add, whole tile: 32 tokens per pass, so that twice as many reads of
      // the residual are in flight per round trip (the last tile's epilogue is not hidden behind
      // any MMA and is pure memory latency).
      bool wide_done = false;
      if constexpr (!GATED && BT >= 128) {
        if (p.tma_out && !part) {                    // the same for every thread
          // tensor memory -> registers -> shared memory (32 tokens x 128 outputs, output index
          // fastest) -> TMA adds the box into the residual.  Nothing is read back, so no memory
          // latency is exposed; two staging buffers, the issuing thread tracks their reads.
          if (threadIdx.x == 64) tma_prefetch_desc(&map_o);
#pragma unroll 1
          for (int c = 0; c < BT; c += 32) {
            if (c >= t_valid) break;
            float v[32];
            tmem_ld16_issue(taddr + c, reinterpret_cast<uint32_t*>(v));
            tmem_ld16_issue(taddr + c + 16, reinterpret_cast<uint32_t*>(v) + 16);
            float* buf = reinterpret_cast<float*>(out_s + ((c >> 5) & 1) * OUT_STAGE_BYTES);
            if (threadIdx.x == 64) bulk_wait_group_read<1>();          // the buffer's last reduce has read it
            asm volatile("bar.sync 1, 128;" ::: "memory");
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) buf[j * TILE_N + n_local] = v[j];
            fence_proxy_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) {
              tma_reduce_add_2d(&map_o, buf, n0, t0 + c);
              bulk_commit_group();
            }
          }
          if (threadIdx.x == 64) {
            if (p.tail_parts > 1 && n_parts > 1) bulk_wait_group<0>();   // the next part adds after this one
            else bulk_wait_group_read<0>();
          }
          wide_done = true;
        }
      }
      if constexpr (!GATED && BT >= 64) {
        if (wide_done) {
        } else
        if (p.mode == MODE_ADD_RESIDUAL && !part && t_valid == BT) {     // the same for every thread
          const bool mine = n < p.N;
#pragma unroll 1
          for (int c = 0; c < BT; c += 32) {
            float v[32], r[32];
            tmem_ld16_issue(taddr + c, reinterpret_cast<uint32_t*>(v));
            tmem_ld16_issue(taddr + c + 16, reinterpret_cast<uint32_t*>(v) + 16);
            float* o = (float*)p.out + (long long)(t0 + c) * p.ldo + n;
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = mine ? o[(long long)j * p.ldo] : 0.f;
            tmem_ld_wait();
            if (mine) {
#pragma unroll
              for (int j = 0; j < 32; ++j) o[(long long)j * p.ldo] = r[j] + v[j];
            }
          }
          wide_done = true;
        }
      }
#pragma unroll 1
      for (int c = 0; !GATED && !wide_done && p.mode != MODE_GATED_SILU && c < BT; c += 16) {
        if (c >= t_valid) break;                     // warp-uniform
        float v[16];
        tmem_ld16(taddr + c, v);
        if (false) {
        } else if (part) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c + j < t_valid) part[(size_t)(c + j) * TILE_N] = v[j];
        } else if (n < p.N) {
          if (p.mode == MODE_ADD_RESIDUAL) {
            // all 16 reads of the residual first, then the 16 writes: one memory round trip
            float* o = (float*)p.out + (long long)(t0 + c) * p.ldo + n;
            float r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = c + j < t_valid ? o[(long long)j * p.ldo] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < t_valid) o[(long long)j * p.ldo] = r[j] + v[j];
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < t_valid) write_out_any(p, t0 + c + j, n, v[j]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
      if (chained) {                                 // the next part's turn; the last part puts the counter back
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) atomicExch(&p.counters[tile], split + 1 == n_parts ? 0 : split + 1);
      }

      if (part) {
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) IERT_TRACE(6);                  // the partial tile is in memory
        const int et = (int)threadIdx.x - 64, c4 = et & 31, tr = et >> 5;
        const float* base = p.ws + ((size_t)tile * p.splits * BT) * TILE_N;
        if (p.coop_reduce) {
          // count in, wait (bounded) until every split of the tile has, add this split's rows
          if (threadIdx.x == 64) {
            atomicAdd(&p.counters[tile], 1);
            int seen = 0;
            for (uint32_t i = 0; i < p.poll_limit; ++i) {
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.counters + tile) : "memory");
              if (seen >= p.splits) break;
              __nanosleep(32);
            }
            *ticket_s = seen >= p.splits ? 1 : 0;
            if (seen < p.splits) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (*ticket_s) {
            const int rows_per = (t_valid + p.splits - 1) / p.splits;
            const int r0 = split * rows_per, r1 = min(t_valid, r0 + rows_per);
            if constexpr (BT > 16) {
              reduce_partial_rows<BT>(p, base, r0 + tr, r1, t0, n0 + c4 * 4, c4, n_idx, scaled ? rstd_s : nullptr);
            } else
            for (int t = r0 + tr; t < r1; t += 4) {        // a token row per 32 threads, 8 splits in flight
              float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int s0 = 0; s0 < p.splits; s0 += 8) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                  v[u] = s0 + u < p.splits
                             ? __ldcg(reinterpret_cast<const float4*>(base + ((size_t)(s0 + u) * BT + t) * TILE_N) + c4)
                             : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 8; ++u) { a.x += v[u].x; a.y += v[u].y; a.z += v[u].z; a.w += v[u].w; }
              }
              write_out4(p, t0 + t, n0 + c4 * 4, a);
            }
          }
          // count out; the last one out zeroes the counter for the next launch
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 64 && atomicAdd(&p.counters[tile], 1) == 2 * p.splits - 1) p.counters[tile] = 0;
        } else {
          if (threadIdx.x == 64) *ticket_s = atomicAdd(&p.counters[tile], 1);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (*ticket_s == p.splits - 1) {             // the last split of this tile: add in split order
            __threadfence();
            reduce_partial_rows<BT>(p, base, tr, t_valid, t0, n0 + c4 * 4, c4, n_idx, scaled ? rstd_s : nullptr);
            if (threadIdx.x == 64) p.counters[tile] = 0;
          }
        }
      }
    }
    if (!ok && lane == 0) {
      if (!*abort_flag) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
      *abort_flag = 1;
    }
  }

  if (threadIdx.x == 64) IERT_TRACE(7);                        // the epilogue warps are done
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, ACC_COLS);
  }
}

// ---- host side ----------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  });
  return fn;
}

struct MapKey {
  const void* ptr; long long rows, cols, ld; int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ (size_t)k.rows;
    h = h * 1000003u ^ (size_t)k.cols;
    h = h * 1000003u ^ (size_t)k.ld;
    return h * 1000003u ^ (size_t)k.box_rows;
  }
};

// A bf16 row-major matrix [rows, cols] with row stride ld, loaded in boxes of box_rows x 64.
bool tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

// The fp32 output [rows, cols] with row stride ld, written in boxes of 32 rows x 128 columns.
bool tensor_map_out(const void* ptr, long long rows, long long cols, long long ld, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, 32};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn || (ld & 3) || ((uintptr_t)ptr & 15)) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)TILE_N, 32};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

// How many token tiles make a group in the order of the tiles (see tile_coords).  With one group
// (all token tiles) the whole activation matrix is read once per weight-row tile unless it stays
// in the L2; with smaller groups the weight matrix is read once per group instead.  A group's
// activations are kept to 32 MB so that they do stay; estimated traffic decides between the two.
// With a prompt of 2,048 tokens the activations of most products fit anyway; with 29,000 tokens
// one group would read them 32 to 112 times.
int token_tiles_per_group(long long x_tile_bytes, long long w_bytes, int n_tiles, int t_tiles) {
  static int off = -1;       // IERT_GEMM_TILE_GROUPS=0: always one group (token tiles fastest)
  if (off < 0) { const char* e = getenv("IERT_GEMM_TILE_GROUPS"); off = (e && e[0] == '0') ? 1 : 0; }
  if (off) return t_tiles;
  const long long keep = 64ll << 20, group_bytes = 32ll << 20;
  const long long x_bytes = x_tile_bytes * t_tiles;
  if (x_bytes <= keep) return t_tiles;
  long long g = group_bytes / (x_tile_bytes > 0 ? x_tile_bytes : 1);
  if (g < 1) g = 1;
  if (g >= t_tiles) return t_tiles;
  const long long groups = (t_tiles + g - 1) / g;
  const long long one_group = x_bytes * n_tiles + w_bytes;
  const long long grouped = (w_bytes <= keep ? w_bytes : w_bytes * groups) + x_bytes;
  return grouped < one_group ? (int)g : t_tiles;
}

bool no_tma_out() {        // IERT_GEMM_TMA_OUT=0: the epilogue reads and writes the residual itself
  static int v = -1;
  if (v < 0) { const char* e = getenv("IERT_GEMM_TMA_OUT"); v = (e && e[0] == '0') ? 1 : 0; }
  return v == 1;
}

bool no_tail_parts() {     // IERT_GEMM_TAIL_PARTS=0: whole tiles only
  static int v = -1;
  if (v < 0) { const char* e = getenv("IERT_GEMM_TAIL_PARTS"); v = (e && e[0] == '0') ? 1 : 0; }
  return v == 1;
}

bool no_coop() {           // IERT_GEMM_COOP=0: the last split of a tile always adds alone
  static int v = -1;
  if (v < 0) { const char* e = getenv("IERT_GEMM_COOP"); v = (e && e[0] == '0') ? 1 : 0; }
  return v == 1;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// Dynamic shared memory of a launch: ring, alignment slack, barriers; the weight-major gated tile
// adds its exchange buffer, the residual add by TMA its two staging buffers.  The one formula for
// the launch and for the estimate of how many CTAs an SM holds (ctas_per_sm_of).
constexpr size_t dynamic_smem_bytes(int stages, int stage_bytes, bool gated_weight_major, bool tma_out, bool row_scales = false) {
  return (size_t)stages * stage_bytes + 1024 + 256 + (gated_weight_major ? XCH_BYTES : row_scales ? 256 + 16 : 0) +
         (tma_out ? 2 * OUT_STAGE_BYTES + 128 : 0);
}

#ifdef IERT_GEMM_TRACE
int g_trace_meta[TRACE_LAUNCHES][8];
int g_trace_next = 0;
#endif

uint32_t g_poll_limit = WAIT_LIMIT;

template <int BT, bool GATED>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, GemmParams p, int grid, cudaStream_t stream,
           const CUtensorMap* mo = nullptr) {
  p.trace_seq = -1;
  p.poll_limit = g_poll_limit;
#ifdef IERT_GEMM_TRACE
  p.trace_seq = g_trace_next % TRACE_LAUNCHES;
  int* tm = g_trace_meta[p.trace_seq];
  tm[0] = g_trace_next++; tm[1] = p.M; tm[2] = p.N; tm[3] = p.K; tm[4] = grid; tm[5] = BT; tm[6] = p.splits; tm[7] = p.mode;
#endif
  constexpr int STAGE_BYTES = (GATED ? 2 : 1) * W_STAGE_BYTES + BT * TILE_K * 2;
  const size_t smem = dynamic_smem_bytes(p.stages, STAGE_BYTES, !GATED && p.mode == MODE_GATED_SILU, p.tma_out != 0,
                                         p.scale.sumsq != nullptr);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<BT, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return iert_check_launch("gemm_tc attribute");
    configured = true;
  }
  launch_dep(gemm_tc_kernel<BT, GATED>, dim3(grid), dim3(THREADS), smem, stream, mw, mx, mo ? *mo : mw, p);
  return iert_check_launch("gemm_tc");
}

// CTAs of the weight-major kernel that one SM holds at once (at most 2 are ever assumed), from
// the kernel's registers, its shared memory and its tensor-memory columns.  The runtime's
// occupancy query is not used: for this kernel it answers 1 whatever the sizes, while two CTAs
// are resident (measured: 256 CTAs that wait for one another finish on 148 SMs).  Should the
// estimate ever be too high, the cooperative reduction's wait runs out and sets the error word.
template <int BT>
int ctas_per_sm_of(int stages) {
  static int cached[13] = {0};
  if (stages < 0 || stages > 12) return 0;
  if (!cached[stages]) {
    // (a plain weight-major launch: no exchange buffer, no TMA-out staging; only such launches reduce cooperatively)
    const size_t smem = dynamic_smem_bytes(stages, W_STAGE_BYTES + BT * TILE_K * 2, false, false, true);   // (the larger of the two plain layouts)
    int n = 0, dev = 0, smem_sm = 0, regs_sm = 0;
    cudaFuncAttributes a;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaFuncGetAttributes(&a, gemm_tc_kernel<BT, false>) == cudaSuccess &&
        cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev) == cudaSuccess) {
      const int regs_per_warp = (((a.numRegs + 7) / 8 * 8) * 32 + 255) / 256 * 256;
      const int by_regs = regs_sm / (regs_per_warp * (THREADS / 32));
      const int by_smem = (int)(smem_sm / (smem + a.sharedSizeBytes + 1024));     // 1 KB reserved per CTA
      const int acc_cols = 2 * BT < 32 ? 32 : 2 * BT;
      const int by_tmem = 512 / acc_cols;
      n = by_regs < by_smem ? by_regs : by_smem;
      if (by_tmem < n) n = by_tmem;
      if (n > 2) n = 2;
    } else {
      cudaGetLastError();
    }
    cached[stages] = n > 0 ? n : -1;
  }
  return cached[stages] > 0 ? cached[stages] : 0;
}

int resident_ctas_per_sm(int bt, int stages) {
  switch (bt) {
    case 16: return ctas_per_sm_of<16>(stages);
    case 32: return ctas_per_sm_of<32>(stages);
    case 64: return ctas_per_sm_of<64>(stages);
    case 128: return ctas_per_sm_of<128>(stages);
    default: return ctas_per_sm_of<256>(stages);
  }
}

}  // namespace

// Bytes of scratch and number of ticket counters a caller should provide.
IERT_API long long iert_gemm_tc_workspace_bytes() { return 48ll << 20; }
IERT_API int iert_gemm_tc_counter_count() { return 8192; }

// x: [M, K] bf16, row stride ldx; w: [N, K] bf16, row stride ldw; out: [M, N] of out_dtype, row
// stride ldo.  mode 0 stores, mode 1 adds into out.  K, ldx and ldw must be multiples of 8
// and the pointers 16-byte aligned (TMA); otherwise IERT_BAD_ARGUMENT is returned and nothing
// is launched.  ws / counters: scratch for split-K, shared by all launches on one stream;
// counters must be zero before the first launch.  force_*: 0 = choose.
namespace {
int gemm_tc_impl(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype,
                 long long ldo, int M, int N, int K, int mode, float* ws, long long ws_bytes,
                 int* counters, int n_counters, int force_bt, int force_splits, int force_stages,
                 const IertRowScale* scale, IertNormAhead* ahead, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IERT_OK;
  if (scale && (!scale->sumsq || scale->parts <= 0 || scale->hidden <= 0 || M > 64)) return IERT_BAD_ARGUMENT;
  if (ahead && (mode != MODE_ADD_RESIDUAL || M > 64 || !ahead->weight || !ahead->scaled_out || !ahead->sumsq_out ||
                (ahead->weight_dtype != IERT_F32 && ahead->weight_dtype != IERT_BF16)))
    return IERT_BAD_ARGUMENT;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return IERT_BAD_ARGUMENT;
  if (mode != MODE_STORE && mode != MODE_ADD_RESIDUAL) return IERT_BAD_ARGUMENT;
  if (out_dtype != IERT_F32 && out_dtype != IERT_BF16) return IERT_BAD_ARGUMENT;
  if (mode == MODE_ADD_RESIDUAL && out_dtype != IERT_F32) return IERT_BAD_ARGUMENT;

  int bt = force_bt;
  // up to 512 tokens 128-token tiles (twice as many of them) beat 256-token tiles with split-K:
  // 512-token prompt 9.7 -> 8.6 ms, 384 tokens 8.7 -> 7.8 ms; from 1,024 tokens on there is no difference
  // Token tile.  65 to 128 tokens: two 64-token tiles (against one 128-token tile: QKV 20 -> 18 us,
  // O 18 -> 16 us; the token-major kernel takes 30 us for the same store).  More tokens: 256-token
  // tiles, split over k while the tiles alone leave SMs empty (256 tokens, K of 14,336: 39 us
  // against 47 us with 64-token tiles); 128-token tiles only where a 256-token tile would be
  // more than half padding.
  // (with a long k the 128-token tiles of 257 to 384 tokens are too many to split and too few to fill the device:
  // 384 tokens, K of 14,336: 87 us, against 71 us for 256-token tiles in two splits)
  if (!bt) bt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 128 ? 64 : (M > 256 && M <= 384 && K < 8192) ? 128 : 256;
  if (bt != 16 && bt != 32 && bt != 64 && bt != 128 && bt != 256) return IERT_BAD_ARGUMENT;

  GemmParams p;
  p.scale = IertRowScale{nullptr, 0, 0, 0.f};
  p.ahead = IertNormAhead{nullptr, 0, nullptr, 0, nullptr, 0};
  if (scale) p.scale = *scale;
  p.tail_parts = 1; p.full_tiles = 0; p.tma_out = 0; p.t_group = 1 << 30;
  p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.mode = mode;
  p.M = M; p.N = N; p.K = K;
  p.ws = ws; p.counters = counters; p.err = err;
  if (!scale && !ahead && !force_bt && !force_splits && ((M > 256 && mode == MODE_STORE) || (M >= 128 && force_stages == -1))) {
    // many tokens, plain store: 128 tokens on the MMA's M side, 256 weight rows on its N side
    // (whole tiles).  Measured on 2,048 tokens: better than weight rows on M for stores (vector
    // stores of a token's row), not for the residual add, which stays on the other kernel.
    if (force_stages == -1) force_stages = 0;
    p.n_step = 2 * TILE_N; p.second_rows = TILE_N;
    p.n_tiles = (N + 2 * TILE_N - 1) / (2 * TILE_N);
    p.t_tiles = (M + 127) / 128;
    p.kb_total = (K + TILE_K - 1) / TILE_K;
    p.splits = 1; p.kb_per_split = p.kb_total; p.coop_reduce = 0;
    p.t_group = token_tiles_per_group(2ll * 128 * K, 2ll * N * K, p.n_tiles, p.t_tiles);
    const int stage_bytes = 2 * W_STAGE_BYTES + 128 * TILE_K * 2;
    int stages = force_stages ? force_stages : (226 * 1024 - 2048) / stage_bytes;
    if (stages < 2 || (size_t)stages * stage_bytes + 1280 > 227 * 1024) return IERT_BAD_ARGUMENT;
    p.stages = stages;
    CUtensorMap mw, mx;
    if (!tensor_map(w, N, K, ldw, TILE_N, &mw) || !tensor_map(x, M, K, ldx, 128, &mx)) return IERT_BAD_ARGUMENT;
    const int tiles = p.n_tiles * p.t_tiles;
    return launch<128, true>(mw, mx, p, tiles < sm_count() ? tiles : sm_count(), stream);
  }
  p.n_step = TILE_N; p.second_rows = 0;
  p.n_tiles = (N + TILE_N - 1) / TILE_N;
  p.t_tiles = (M + bt - 1) / bt;
  p.kb_total = (K + TILE_K - 1) / TILE_K;
  p.t_group = token_tiles_per_group(2ll * bt * K, 2ll * N * K, p.n_tiles, p.t_tiles);
  const int tiles = p.n_tiles * p.t_tiles;
  const int stage_bytes = W_STAGE_BYTES + bt * TILE_K * 2;
  const int ctas_per_sm = bt <= 64 ? 2 : 1;
  const int slots = sm_count() * ctas_per_sm;
  const int smem_budget = (ctas_per_sm == 2 ? 113 : 226) * 1024 - 2048;
  int stages = force_stages ? force_stages : smem_budget / stage_bytes;
  if (stages > 12) stages = 12;
  if (stages < 2 || (size_t)stages * stage_bytes + 1280 > 227 * 1024) return IERT_BAD_ARGUMENT;
  p.stages = stages;

  int splits = 1;
  if (force_splits) {
    splits = force_splits;
  } else if (tiles * 2 <= slots) {
    // As many splits as fill the CTA slots (two CTAs per SM up to 64-token tiles: they hide each
    // other's start-up and epilogue).  Measured in whole decoding steps at 7B layer sizes against
    // one CTA per SM with a ring as deep as shared memory allows: equal at batch 64, 2 % faster
    // at batch 32, 5 % at batch 8.
    splits = slots / tiles;
    const int max_by_k = p.kb_total / 4 > 0 ? p.kb_total / 4 : 1;     // at least 4 k-blocks per split
    if (splits > max_by_k) splits = max_by_k;
    const int cap = bt >= 32 ? 8 : 16;                  // partial tiles grow with the token tile
    if (splits > cap) splits = cap;
  }
  if (splits < 1) splits = 1;
  if (splits > p.kb_total) splits = p.kb_total;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;        // no empty split
  if (splits > 1) {
    const long long need = (long long)tiles * splits * bt * TILE_N * 4;
    if (!ws || !counters || need > ws_bytes || tiles > n_counters) {
      if (force_splits) return IERT_BAD_ARGUMENT;
      splits = 1;
      p.kb_per_split = p.kb_total;
    }
  }
  p.splits = splits;
  // row scales and the next norm's first half are the split-K reduction's work, on tiles of 32 or 64 tokens
  if ((scale || ahead) && (splits < 2 || bt < 32 || bt > 64)) return IERT_BAD_ARGUMENT;
  if (ahead) {
    ahead->parts = (N + TILE_N - 1) / TILE_N;
    p.ahead = *ahead;
  }
  const int total_work = tiles * splits;
  if (!force_stages && ctas_per_sm == 2 && total_work <= sm_count()) {
    // every CTA has an SM to itself: let its ring use the whole shared memory
    stages = (226 * 1024 - 2048) / stage_bytes;
    if (stages > 12) stages = 12;
    p.stages = stages;
  }

  CUtensorMap mw, mx, mo;
  if (!tensor_map(w, N, K, ldw, TILE_N, &mw) || !tensor_map(x, M, K, ldx, bt, &mx)) return IERT_BAD_ARGUMENT;
  // Many tokens, residual add: the epilogue hands its tile to TMA, which adds it into the residual
  // (no read of the residual by the SM).  Needs two staging buffers beside the ring.
  if (mode == MODE_ADD_RESIDUAL && bt >= 128 && splits == 1 && !no_tma_out() && tensor_map_out(out, M, N, ldo, &mo)) {
    int st = stages;
    while (st >= 2 && (size_t)st * stage_bytes + 1280 + 2 * OUT_STAGE_BYTES + 128 > 227 * 1024) --st;
    if (st >= 2 && (force_stages <= 0 || st == stages)) { p.tma_out = 1; stages = st; p.stages = st; }
  }
  int grid = total_work < slots ? total_work : slots;
  // The splits of a tile may wait for one another only if every CTA of the grid is resident.  Residency is
  // estimated (resident_ctas_per_sm) from the registers, the tensor memory and the shared memory of a PLAIN
  // weight-major launch: no gated tile (that is another entry point) and no residual add by TMA (that needs
  // splits == 1, the cooperative reduction splits > 1).  A variant that breaks this must not reduce
  // cooperatively, or its waits could expire: refuse it here rather than find out on the device.
  p.coop_reduce = splits > 1 && !no_coop() && total_work <= grid &&
                  grid <= sm_count() * resident_ctas_per_sm(bt, stages);
  if (p.coop_reduce && (p.tma_out || p.mode == MODE_GATED_SILU || p.tail_parts > 1)) return IERT_BAD_ARGUMENT;
  // Residual adds over many tokens whose tiles leave the last wave part empty: the tiles of that
  // wave are cut into parts of k (see WorkIter).  One CTA per SM; parts chosen to fill the SMs.
  if (!force_splits && !no_tail_parts() && splits == 1 && mode == MODE_ADD_RESIDUAL && bt >= 128 && ctas_per_sm == 1 &&
      counters && tiles <= n_counters && tiles > sm_count() && tiles % sm_count() != 0) {
    const int sms = sm_count(), n_tail = tiles % sms;
    int best = 1;
    double best_cost = 1.0;                            // the last wave in units of a whole tile
    for (int parts = 2; parts <= 8; ++parts) {
      // A part's epilogue (a few us) has to stay short beside its MMAs, and the parts of a tile add
      // one after the other: measured, parts pay from about 40 k-blocks each on (K of 14,336 in
      // four parts: 189 -> 179 us), and cost time below that (K of 4,096: 59 -> 62 us).
      if (p.kb_total / parts < 40) break;
      const double cost = (double)((n_tail * parts + sms - 1) / sms) / parts + 0.02 * parts;
      if (cost < best_cost) { best_cost = cost; best = parts; }
    }
    if (best > 1) {
      p.tail_parts = best;
      p.full_tiles = tiles - n_tail;
      grid = sms;
    }
  }
  switch (bt) {
    case 16: return launch<16, false>(mw, mx, p, grid, stream);
    case 32: return launch<32, false>(mw, mx, p, grid, stream);
    case 64: return launch<64, false>(mw, mx, p, grid, stream);
    case 128: return launch<128, false>(mw, mx, p, grid, stream, p.tma_out ? &mo : nullptr);
    default: return launch<256, false>(mw, mx, p, grid, stream, p.tma_out ? &mo : nullptr);
  }
}
}  // namespace

#ifdef IERT_GEMM_TRACE
// stamps: [64][304][8] unsigned 64-bit; meta: [64][8] int (sequence number, M, N, K, grid, token tile, splits, mode)
IERT_API int iert_gemm_tc_trace_read(unsigned long long* stamps, int* meta) {
  if (cudaMemcpyFromSymbol(stamps, g_tc_trace, sizeof(unsigned long long) * TRACE_LAUNCHES * TRACE_CTAS * TRACE_EVENTS) != cudaSuccess)
    return IERT_CUDA_ERROR;
  memcpy(meta, g_trace_meta, sizeof(g_trace_meta));
  return IERT_OK;
}
#endif

// How many times a CTA polls its tile's counter before it gives up waiting for the tile's other CTAs (default
// 2^22, about a second; 0 restores the default).  For tests that let such a wait run out: the kernel then sets
// IERT_ERR_WAIT_EXPIRED in the error word, skips the work that depended on the wait and ends like any other.
IERT_API void iert_gemm_tc_set_poll_limit(unsigned int polls) { g_poll_limit = polls ? polls : WAIT_LIMIT; }

IERT_API int iert_gemm_tc(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype,
                          long long ldo, int M, int N, int K, int mode, float* ws, long long ws_bytes,
                          int* counters, int n_counters, int force_bt, int force_splits, int force_stages,
                          int* err, cudaStream_t stream) {
  return gemm_tc_impl(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, mode, ws, ws_bytes, counters, n_counters, force_bt,
                      force_splits, force_stages, nullptr, nullptr, err, stream);
}

// The same for one-token steps of 17 to 64 tokens whose input or output takes part in an RMSNorm split around
// the kernel boundary (see common.cuh):
//   scale (optional)  x is a norm's first half: the outputs are multiplied by each row's 1 / rms;
//   ahead (optional; mode 1)  the reduction also writes the next norm's first half; ahead->parts is set to
//                     the number of partial sums per row (one per tile of 128 columns).
// Both are the split-K reduction's work: IERT_BAD_ARGUMENT, nothing launched, where a launch would not split k
// or its token tile is not 32 or 64.
IERT_API int iert_gemm_tc_scaled(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype,
                                 long long ldo, int M, int N, int K, int mode, float* ws, long long ws_bytes,
                                 int* counters, int n_counters, const IertRowScale* scale, IertNormAhead* ahead,
                                 int force_bt, int force_splits, int* err, cudaStream_t stream) {
  return gemm_tc_impl(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, mode, ws, ws_bytes, counters, n_counters, force_bt,
                      force_splits, 0, scale, ahead, err, stream);
}

// act[t, i] = silu(x[t] . w[i]) * (x[t] . w[inter + i]) for w = [gate; up] of 2 * inter rows,
// in one kernel (two accumulators per tile).  act: bf16 [M, inter], row stride ldo.  Whole
// tiles only; same alignment rules as iert_gemm_tc.
namespace {
int gemm_tc_gated_impl(const void* x, long long ldx, const void* w, long long ldw, void* act,
                       long long ldo, int M, int inter, int K, const IertRowScale* scale, int force_bt, int force_stages,
                       int* err, cudaStream_t stream) {
  if (M <= 0 || inter <= 0) return IERT_OK;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return IERT_BAD_ARGUMENT;
  if (scale && (!scale->sumsq || scale->parts <= 0 || scale->hidden <= 0)) return IERT_BAD_ARGUMENT;
  GemmParams p;
  p.scale = IertRowScale{nullptr, 0, 0, 0.f};
  p.tail_parts = 1; p.full_tiles = 0; p.tma_out = 0; p.t_group = 1 << 30;
  p.out = act; p.ldo = ldo; p.out_dtype = IERT_BF16; p.mode = MODE_GATED_SILU;
  p.M = M; p.N = inter; p.K = K;
  const bool weight_major = force_bt ? (force_bt != 128 && M <= force_bt)
                                     : (M <= 64 && (inter + TILE_N / 2 - 1) / (TILE_N / 2) >= sm_count());
  if (force_bt && force_bt != 16 && force_bt != 32 && force_bt != 64 && force_bt != 128) return IERT_BAD_ARGUMENT;
  if (force_bt && force_bt != 128 && M > force_bt) return IERT_BAD_ARGUMENT;
  if (weight_major) {
    // Few tokens (decoding): weight rows on the MMA's M side, 64 gate rows and their 64 up rows
    // per tile, no split over k.  Chosen when its tiles alone fill the device; for smaller
    // matrices the caller does better with the split product and a separate activation.
    const int wbt = force_bt ? force_bt : (M <= 16 ? 16 : M <= 32 ? 32 : 64);
    p.n_step = TILE_N / 2; p.second_rows = inter;
    p.n_tiles = (inter + TILE_N / 2 - 1) / (TILE_N / 2);
    p.t_tiles = 1;
    p.kb_total = (K + TILE_K - 1) / TILE_K;
    p.splits = 1; p.kb_per_split = p.kb_total; p.coop_reduce = 0;
    p.ws = nullptr; p.counters = nullptr; p.err = err;
    if (scale) p.scale = *scale;
    const int stage_bytes = W_STAGE_BYTES + wbt * TILE_K * 2;
    int stages = force_stages ? force_stages : (113 * 1024 - 2048 - XCH_BYTES) / stage_bytes;
    if (stages > 12) stages = 12;
    if (stages < 2 || (size_t)stages * stage_bytes + 1280 + XCH_BYTES > 227 * 1024) return IERT_BAD_ARGUMENT;
    p.stages = stages;
    CUtensorMap mw, mx;
    if (!tensor_map(w, 2ll * inter, K, ldw, TILE_N / 2, &mw) || !tensor_map(x, M, K, ldx, wbt, &mx)) return IERT_BAD_ARGUMENT;
    const int slots = 2 * sm_count();
    const int grid = p.n_tiles < slots ? p.n_tiles : slots;
    switch (wbt) {
      case 16: return launch<16, false>(mw, mx, p, grid, stream);
      case 32: return launch<32, false>(mw, mx, p, grid, stream);
      default: return launch<64, false>(mw, mx, p, grid, stream);
    }
  }
  if (scale) return IERT_BAD_ARGUMENT;                 // only the one-token form scales its rows
  const int bt = 128;                                  // tokens per tile: the MMA's M side
  p.n_step = TILE_N; p.second_rows = inter;
  p.n_tiles = (inter + TILE_N - 1) / TILE_N;
  p.t_tiles = (M + bt - 1) / bt;
  p.kb_total = (K + TILE_K - 1) / TILE_K;
  p.splits = 1; p.kb_per_split = p.kb_total; p.coop_reduce = 0;
  p.ws = nullptr; p.counters = nullptr; p.err = err;
  p.t_group = token_tiles_per_group(2ll * bt * K, 4ll * inter * K, p.n_tiles, p.t_tiles);
  const int tiles = p.n_tiles * p.t_tiles;
  const int stage_bytes = 2 * W_STAGE_BYTES + bt * TILE_K * 2;
  const int slots = sm_count();
  const int smem_budget = 226 * 1024 - 2048;
  int stages = force_stages ? force_stages : smem_budget / stage_bytes;
  if (stages > 12) stages = 12;
  if (stages < 2 || (size_t)stages * stage_bytes + 1280 > 227 * 1024) return IERT_BAD_ARGUMENT;
  p.stages = stages;
  CUtensorMap mw, mx;
  if (!tensor_map(w, 2ll * inter, K, ldw, TILE_N, &mw) || !tensor_map(x, M, K, ldx, bt, &mx)) return IERT_BAD_ARGUMENT;
  const int grid = tiles < slots ? tiles : slots;
  return launch<128, true>(mw, mx, p, grid, stream);
}
}  // namespace

IERT_API int iert_gemm_tc_gated(const void* x, long long ldx, const void* w, long long ldw, void* act,
                                long long ldo, int M, int inter, int K, int force_bt, int force_stages,
                                int* err, cudaStream_t stream) {
  return gemm_tc_gated_impl(x, ldx, w, ldw, act, ldo, M, inter, K, nullptr, force_bt, force_stages, err, stream);
}

// The one-token form (M <= 64) for an x that is the first half of an RMSNorm (IertNormAhead of the kernel
// that wrote it): gate and up are multiplied by each row's 1 / rms before the activation.
// IERT_BAD_ARGUMENT, nothing launched, where the one-token form does not apply.
IERT_API int iert_gemm_tc_gated_scaled(const void* x, long long ldx, const void* w, long long ldw, void* act,
                                       long long ldo, int M, int inter, int K, const IertRowScale* scale, int force_bt,
                                       int* err, cudaStream_t stream) {
  if (!scale) return IERT_BAD_ARGUMENT;
  return gemm_tc_gated_impl(x, ldx, w, ldw, act, ldo, M, inter, K, scale, force_bt, 0, err, stream);
}
