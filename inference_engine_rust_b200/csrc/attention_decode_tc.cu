// Decode attention on the tensor cores: one query token per sequence against the paged cache,
// split over the keys, bf16 operands (mma.sync m16n8k16), fp32 scores / softmax / output.
// Compiled once per head size (-DHEAD_DIM, multiple of 16 up to 256), like the prompt kernel.
//
//   grid (kv_heads * slices, sequences, splits).  The up to 16 query heads that share one kv
//   head are the 16 rows of the MMA tile, so every key and value is read once per group and
//   the arithmetic is a handful of MMAs per page: the kernel is a stream of page loads.
//   A CTA walks its share of the sequence's 64-position pages; each page's keys and values
//   (two contiguous runs of 64 * HEAD_DIM bf16) are fetched with cp.async into a three-deep ring
//   of shared memory with padded rows (conflict-free ldmatrix); rows outside [j_min, pos] are
//   zero-filled, so memory that was never written cannot reach the arithmetic.
//   Each of the 4 warps takes 16 of a page's 64 keys with its own running maximum and sum;
//   the warps are merged through shared memory in warp order at the end, and the split's
//   partial result (unnormalised output, maximum, sum) goes to scratch memory.  A second
//   kernel merges the splits in split order; a single split writes the output itself.
//
// Optionally the rotary position encoding and the cache write of the step are part of this
// kernel (angle pos * theta^(-2k/d) in fp32, src/ops/rope.rs:40-57; rotate, then store, then
// attend, src/layers/attention.rs:577-606): every CTA rotates its group's queries as it stages
// them; the CTA that owns the newest page rotates the new key, puts the new key and value row
// into that page's tile in shared memory, and (one CTA per kv head) writes both to the cache.
//
// Visible keys: [max(0, pos + 1 - W), pos] (src/layers/attention.rs:609-613); scale from the
// caller; softmax in fp32 (src/ops/softmax.rs:11-25).
#include "common.cuh"
#include "sm100.cuh"
#include "tma_host.cuh"

#include <cstdlib>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16>"
#endif

using namespace iert;

namespace {

constexpr int HD = HEAD_DIM;
constexpr int PAGE = 64, WARPS = 4, THREADS = WARPS * 32, ROWS = 16;
constexpr int ROW_BYTES = HD * 2 + 16;
constexpr int TILE_BYTES = PAGE * ROW_BYTES;
constexpr int KSTEPS = HD / 16;
constexpr int NSTAGE = 3;                       // pages in flight per CTA: the one in use and two behind it

struct DecodeTcParams {
  const __nv_bfloat16* qkv;   // [T, (heads + 2 kv_heads) * HD], queries rotated
  float* part_out;            // [T, heads, splits, HD]
  float* part_ml;             // [T, heads, splits, 2]  (maximum in base-2 units, sum)
  __nv_bfloat16* out;         // [T, heads * HD]
  int heads, splits, slices, gt;
  int target_ctas;            // > 0: a sequence is cut into as many of the `splits` parts as its length asks for
  float scale_log2e;
  int* err;
  // Fused position encoding (rope != 0): `qkv` comes straight from the projection; the kernel
  // rotates the queries and the new key itself and, if store != 0, writes the new key and
  // value into the cache.  With rope == 0 the kernel before has done all of that.
  const float* inv_freq;      // [rotary_dim / 2]
  int rope, rotary_dim, pairing, store;
};

__device__ __forceinline__ void cp16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One page's rows [0, 64) of one kv head into a padded tile; rows outside [lo, hi] are zeros.
__device__ __forceinline__ void load_page(uint8_t* tile, const __nv_bfloat16* src, int lo, int hi) {
  constexpr int CHUNKS = HD / 8;
  for (int i = threadIdx.x; i < PAGE * CHUNKS; i += THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const bool ok = r >= lo && r <= hi;
    cp16(tile + r * ROW_BYTES + c * 16, src + (ok ? r * HD + c * 8 : 0), ok);
  }
}

// Pages of keys a one-token step of sequence s reads (0 for a padding sequence).
__device__ __forceinline__ int pages_of_sequence(const IertBatchView& b, const IertKvView& c, int s) {
  if (b.slot_ids[s] < 0) return 0;
  const int pos = b.pos0[s] + (b.cu_q[s + 1] - b.cu_q[s]) - 1;
  const int j_min = c.window > 0 ? max(0, pos + 1 - c.window) : 0;
  return pos / PAGE + 1 - j_min / PAGE;
}

// Into how many parts a sequence of `my_pages` pages is cut when the sequences of the step have
// unequal lengths: every part should hold about total pages / target CTAs, so that a long sequence
// gets many short parts and a short one a single part, and the step ends when the average CTA
// does rather than when the longest sequence's CTAs do.  Every CTA of the step computes the same
// numbers from the step's description (whole block; `red`: shared scratch of blockDim / 32 ints).
__device__ int balanced_parts(const IertBatchView& b, const IertKvView& c, int my_pages, int max_parts,
                              int target_ctas, int ctas_per_sequence_part, int* red) {
  int tot = 0;
  for (int s = threadIdx.x; s < b.n_seqs; s += blockDim.x) tot += pages_of_sequence(b, c, s);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = tot;
  __syncthreads();
  tot = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
  __syncthreads();
  const long long units = (long long)tot * ctas_per_sequence_part;
  const int per_part = (int)max(1ll, (units + target_ctas - 1) / target_ctas);
  return max(1, min(max_parts, (my_pages + per_part - 1) / per_part));
}

__global__ void __launch_bounds__(THREADS)
attention_decode_tc_kernel(DecodeTcParams p, IertBatchView b, IertKvView c) {
  extern __shared__ __align__(16) uint8_t smem[];
  auto k_tile = [&](int i) { return smem + (size_t)(2 * i) * TILE_BYTES; };
  auto v_tile = [&](int i) { return smem + (size_t)(2 * i + 1) * TILE_BYTES; };
  uint8_t* q_tile = smem + 2 * NSTAGE * TILE_BYTES;      // [16][ROW_BYTES]
  float* cs_tab = reinterpret_cast<float*>(q_tile + ROWS * ROW_BYTES);   // [HD / 2] cos, [HD / 2] sin (fused rope)
  __nv_bfloat16* new_kv = reinterpret_cast<__nv_bfloat16*>(cs_tab + HD);  // [2][HD]: the step's own key and value

  pdl_launch_dependents();     // the next kernel may start its preamble now
  // The kernel before this one wrote the queries and the newest key and value; the step's
  // description, the page table and every older page are in place already.  So a CTA whose
  // first pages are older than the newest one starts fetching them before it waits for that
  // kernel.
  const int split = blockIdx.z, t = blockIdx.y;      // parts slowest: CTAs of parts a sequence does not use start last
  const int kvh = blockIdx.x / p.slices, slice = blockIdx.x % p.slices;
  const int group = p.heads / c.kv_heads;
  const int g0 = slice * p.gt;
  const int n_g = min(p.gt, group - g0);
  const int head0 = kvh * group + g0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;

  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  float* po = p.part_out + (((size_t)t * p.heads + head0) * p.splits + split) * HD;
  float* pml = p.part_ml + (((size_t)t * p.heads + head0) * p.splits + split) * 2;
  if (slot < 0) {
    pdl_wait();                // the scratch may still be read by an earlier kernel's successor
    if (p.splits == 1) {       // a padding sequence: zeros
      for (int i = threadIdx.x; i < n_g * HD; i += THREADS)
        p.out[((size_t)t * p.heads + head0) * HD + i] = __float2bfloat16_rn(0.f);
    } else if (threadIdx.x < n_g) {
      pml[(size_t)threadIdx.x * p.splits * 2] = -INFINITY; pml[(size_t)threadIdx.x * p.splits * 2 + 1] = 0.f;
    }
    return;
  }
  const int pos = b.pos0[s] + (t - b.cu_q[s]);
  const int j_min = c.window > 0 ? max(0, pos + 1 - c.window) : 0;
  const int pg_lo = j_min / PAGE, pg_hi = pos / PAGE + 1;           // logical pages [pg_lo, pg_hi)
  int n_splits = p.splits;
  if (p.target_ctas > 0 && p.splits > 1) {
    __shared__ int red[WARPS];
    n_splits = balanced_parts(b, c, pg_hi - pg_lo, p.splits, p.target_ctas, gridDim.x, red);
    if (split >= n_splits) return;                     // this sequence is cut into fewer parts
  }
  const int per = (pg_hi - pg_lo + n_splits - 1) / n_splits;
  const int my_lo = pg_lo + split * per, my_hi = min(pg_hi, my_lo + per);

  // this CTA's range holds the newest page and the kernel has to supply the newest row itself
  const bool own_new_row = p.rope && p.store && my_lo < my_hi && my_hi == pg_hi;
  const int half = p.rotary_dim / 2;
  if (p.rope) {                                          // angles: no dependency on the kernel before
    for (int k = threadIdx.x; k < half; k += THREADS) {
      float sn, cs_;
      sincosf((float)pos * p.inv_freq[k], &sn, &cs_);
      cs_tab[k] = cs_;
      cs_tab[half + k] = sn;
    }
  }
  auto issue = [&](int pg, int buf) {
    const int page = c.page_table[(size_t)slot * c.table_width + pg % c.ring_pages];
    const bool ok = page >= 0 && page < c.n_pages;
    if (!ok && threadIdx.x == 0) atomicOr(p.err, IERT_ERR_PAGE_RANGE);
    const size_t off = (((size_t)(ok ? page : 0) * c.kv_heads + kvh) * PAGE) * HD;
    const int lo = ok ? max(0, j_min - pg * PAGE) : PAGE;
    int hi = ok ? min(PAGE - 1, pos - pg * PAGE) : -1;
    if (own_new_row && pg == pos / PAGE) --hi;           // the newest row comes from the projection, below
    load_page(k_tile(buf), (const __nv_bfloat16*)c.k + off, lo, hi);
    load_page(v_tile(buf), (const __nv_bfloat16*)c.v + off, lo, hi);
  };
  // queries of the group: rows 0..n_g-1 of a 16-row tile, the other rows zero
  const __nv_bfloat16* tok_row = p.qkv + (size_t)t * ((size_t)(p.heads + 2 * c.kv_heads) * HD);
  // v[i0], v[i1] of a head rotated by the angle of pair k, fp32 math, bf16 out
  auto rotate_into = [&](const __nv_bfloat16* src, __nv_bfloat16* dst, int k) {
    const int i0 = p.pairing == IERT_PAIR_HALF ? k : 2 * k;
    const int i1 = p.pairing == IERT_PAIR_HALF ? k + half : 2 * k + 1;
    const float a = __bfloat162float(src[i0]), bb = __bfloat162float(src[i1]);
    dst[i0] = __float2bfloat16_rn(a * cs_tab[k] - bb * cs_tab[half + k]);
    dst[i1] = __float2bfloat16_rn(a * cs_tab[half + k] + bb * cs_tab[k]);
  };
  auto load_queries = [&]() {
    const __nv_bfloat16* q = tok_row + (size_t)head0 * HD;
    if (p.rope) {
      __syncthreads();                                   // the angle table is complete
      for (int i = threadIdx.x; i < ROWS * (HD / 2); i += THREADS) {
        const int r = i / (HD / 2), k = i % (HD / 2);
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(q_tile + r * ROW_BYTES);
        if (r >= n_g) { dst[2 * k] = __float2bfloat16_rn(0.f); dst[2 * k + 1] = __float2bfloat16_rn(0.f); }
        else if (k < half) rotate_into(q + r * HD, dst, k);
        else {                                           // dimensions beyond rotary_dim pass through
          const int d = p.rotary_dim + 2 * (k - half);
          dst[d] = q[r * HD + d]; dst[d + 1] = q[r * HD + d + 1];
        }
      }
      return;
    }
    constexpr int CHUNKS = HD / 8;
    for (int i = threadIdx.x; i < ROWS * CHUNKS; i += THREADS) {
      const int r = i / CHUNKS, cc = i % CHUNKS;
      cp16(q_tile + r * ROW_BYTES + cc * 16, q + (r < n_g ? r * HD + cc * 8 : 0), r < n_g);
    }
  };
  // One commit group per page, empty groups included, in the order of use, so that "all but
  // the newest NSTAGE - 1 groups have landed" always means "the page about to be used has
  // landed".  The queries travel in the first group, or, with `early`, in a group of their own
  // behind the first pages.  `early`: none of the first NSTAGE - 1
  // pages is the newest page (whose last row the kernel before this one writes), and a page of
  // a ring cannot be overwritten while it is read (the newest key lands in the newest page).
  const bool early = my_lo + NSTAGE - 1 <= pos / PAGE;
  if (!early) pdl_wait();
  if (!early) load_queries();
#pragma unroll
  for (int i = 0; i < NSTAGE - 1; ++i) {
    if (my_lo + i < my_hi) issue(my_lo + i, i);
    cp_commit();
  }
  if (early) {
    pdl_wait();
    load_queries();              // a group of their own, younger than the first pages: see the first wait
    cp_commit();
  }
  if (own_new_row) {
    // the new key (rotated) and value: staged for the newest page's tile and, once per kv
    // head, written to the cache (src/layers/attention.rs:604-606)
    const __nv_bfloat16* kn = tok_row + (size_t)(p.heads + kvh) * HD;
    const __nv_bfloat16* vn = tok_row + (size_t)(p.heads + c.kv_heads + kvh) * HD;
    for (int k = threadIdx.x; k < HD / 2; k += THREADS) {
      if (k < half) rotate_into(kn, new_kv, k);
      else { const int d = p.rotary_dim + 2 * (k - half); new_kv[d] = kn[d]; new_kv[d + 1] = kn[d + 1]; }
      new_kv[HD + 2 * k] = vn[2 * k];
      new_kv[HD + 2 * k + 1] = vn[2 * k + 1];
    }
    __syncthreads();
    if (slice == 0) {
      const int page = c.page_table[(size_t)slot * c.table_width + (pos / PAGE) % c.ring_pages];
      if (page >= 0 && page < c.n_pages) {
        const size_t off = ((((size_t)page * c.kv_heads + kvh) * PAGE) + pos % PAGE) * HD;
        for (int d = threadIdx.x; d < HD; d += THREADS) {
          ((__nv_bfloat16*)c.k)[off + d] = new_kv[d];
          ((__nv_bfloat16*)c.v)[off + d] = new_kv[HD + d];
        }
      } else if (threadIdx.x == 0) {
        atomicOr(p.err, IERT_ERR_PAGE_RANGE);
      }
    }
  }

  uint32_t qf[KSTEPS][4];
  float o[KSTEPS * 2][4];
#pragma unroll
  for (int n = 0; n < KSTEPS * 2; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_row = -INFINITY, l_row = 0.f;          // row g (a head of the group); rows >= 8 are padding

  for (int pg = my_lo; pg < my_hi; ++pg) {
    const int buf = (pg - my_lo) % NSTAGE;
    if (pg + NSTAGE - 1 < my_hi) issue(pg + NSTAGE - 1, (pg - my_lo + NSTAGE - 1) % NSTAGE);
    cp_commit();
    if (early && pg == my_lo) cp_wait<1>();      // the queries' group is the second youngest here
    else cp_wait<NSTAGE - 1>();
    __syncthreads();
    if (own_new_row && pg == pos / PAGE) {               // the newest row of the newest page
      const int r = pos % PAGE;
      for (int d = threadIdx.x; d < HD; d += THREADS) {
        reinterpret_cast<__nv_bfloat16*>(k_tile(buf) + r * ROW_BYTES)[d] = new_kv[d];
        reinterpret_cast<__nv_bfloat16*>(v_tile(buf) + r * ROW_BYTES)[d] = new_kv[HD + d];
      }
      __syncthreads();
    }
    if (pg == my_lo) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldsm4(qf[ks], q_tile + (lane & 15) * ROW_BYTES + (ks * 16 + (lane >> 4) * 8) * 2);
    }
    // ---- scores of this warp's 16 keys: S[16 rows][16 keys]
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t kb[4];
      ldsm4(kb, k_tile(buf) + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * ROW_BYTES + (ks * 16 + ((lane >> 3) & 1) * 8) * 2);
      mma16816(sc[0], qf[ks], kb[0], kb[1]);
      mma16816(sc[1], qf[ks], kb[2], kb[3]);
    }
    // ---- mask and running softmax for row g (elements 0,1 of each tile; 2,3 belong to row g+8)
    const int jbase = pg * PAGE + warp * 16;
    float mx = m_row;
    float v[2][2];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = jbase + n * 8 + tq * 2 + e;
        v[n][e] = (j >= j_min && j <= pos) ? sc[n][e] * p.scale_log2e : -INFINITY;
        mx = fmaxf(mx, v[n][e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float alpha = m_row == -INFINITY ? 0.f : exp2f(m_row - mx);
    m_row = mx;
    l_row *= alpha;
    float pr[2][2];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[n][e] = (v[n][e] == -INFINITY || mx == -INFINITY) ? 0.f : exp2f(v[n][e] - mx);
        l_row += pr[n][e];
      }
#pragma unroll
    for (int n = 0; n < KSTEPS * 2; ++n) { o[n][0] *= alpha; o[n][1] *= alpha; }
    // ---- O += P V over the warp's 16 keys (rows g+8 of P are zero)
    const uint32_t pa[4] = {pack2(pr[0][0], pr[0][1]), 0u, pack2(pr[1][0], pr[1][1]), 0u};
#pragma unroll
    for (int dp = 0; dp < KSTEPS; ++dp) {
      uint32_t vb[4];
      ldsm4t(vb, v_tile(buf) + (warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * ROW_BYTES + (dp * 16 + (lane >> 4) * 8) * 2);
      mma16816(o[2 * dp], pa, vb[0], vb[1]);
      mma16816(o[2 * dp + 1], pa, vb[2], vb[3]);
    }
    __syncthreads();
  }

  // ---- merge the four warps in warp order (shared memory is free now), write the partial
  cp_wait<0>();
  __syncthreads();
  l_row += __shfl_xor_sync(0xffffffffu, l_row, 1);
  l_row += __shfl_xor_sync(0xffffffffu, l_row, 2);
  float* o_s = reinterpret_cast<float*>(smem);                 // [WARPS][8][HD]
  float* ml_s = o_s + WARPS * 8 * HD;                          // [WARPS][8][2]
#pragma unroll
  for (int n = 0; n < KSTEPS * 2; ++n) {
    o_s[(warp * 8 + g) * HD + n * 8 + tq * 2] = o[n][0];
    o_s[(warp * 8 + g) * HD + n * 8 + tq * 2 + 1] = o[n][1];
  }
  if (tq == 0) { ml_s[(warp * 8 + g) * 2] = m_row; ml_s[(warp * 8 + g) * 2 + 1] = l_row; }
  __syncthreads();
  const bool direct = p.splits == 1;                  // a single split: its result is the output
  for (int r = 0; r < n_g && r < 8; ++r) {
    float mm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, ml_s[(w * 8 + r) * 2]);
    float wgt[WARPS], ll = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      const float mw = ml_s[(w * 8 + r) * 2];
      wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      ll += wgt[w] * ml_s[(w * 8 + r) * 2 + 1];
    }
    const float inv = ll > 0.f ? 1.0f / ll : 0.f;
    for (int d = threadIdx.x; d < HD; d += THREADS) {
      float acc = 0.f;
      for (int w = 0; w < WARPS; ++w) acc += wgt[w] * o_s[(w * 8 + r) * HD + d];
      if (direct) p.out[((size_t)t * p.heads + head0 + r) * HD + d] = __float2bfloat16_rn(acc * inv);
      else po[(size_t)r * p.splits * HD + d] = acc;
    }
    if (!direct && threadIdx.x == 0) { pml[(size_t)r * p.splits * 2] = mm; pml[(size_t)r * p.splits * 2 + 1] = ll; }
  }
}

#if HEAD_DIM % 64 == 0
// ---------------------------------------------------------------------------------------------
// The same kernel with the pages brought in by TMA (head sizes that are multiples of 64).  A
// fifth warp is the producer: one thread waits for a ring slot to be empty, arms its barrier and
// asks for the page's keys and values as boxes of 64 positions x 64 dimensions, written to shared
// memory with the 128-byte swizzle (no padding: ldmatrix is conflict-free through the swizzle).
// The four consumer warps wait for a slot's barrier, each uses its own 16 positions of the page
// and arrives on the slot's "empty" barrier: no block-wide barrier inside the loop over pages,
// and no load instructions in the warps that compute.  TMA brings whole pages, so positions
// outside [j_min, pos] hold whatever the page held before: their scores are masked as before
// (a select, so not even NaN gets through), and each warp zeroes its own rows of the values
// that are out of range before it multiplies by them (0 x NaN would be NaN).  Every wait on a
// barrier is bounded.  When one runs out, the warp that saw it records the fault and raises a flag
// in shared memory that every other wait of the CTA polls: the producer stops asking for pages,
// the consumers leave the loop over pages, one thread then waits (bounded again) until the
// producer has stopped and every copy it had asked for has landed, and only then does the CTA
// touch the ring again: it skips the merge and writes an empty partial result (maximum -inf, sum
// 0; zeros if it is the only part), so that nothing stale is mixed in.
constexpr int TMA_THREADS = THREADS + 32;
constexpr int BOX_BYTES = PAGE * 128;                   // 64 positions x 64 dimensions of bf16
constexpr int BOXES = HD / 64;
constexpr int TMA_TILE_BYTES = BOXES * BOX_BYTES;       // one page's keys (or values) of one kv head

// Address of the 16-byte chunk holding dimensions [col, col + 8) of position `row` in a swizzled tile.
__device__ __forceinline__ uint8_t* swz(uint8_t* tile, int row, int col) {
  return tile + (col >> 6) * BOX_BYTES + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4);
}

// Bounded wait that gives up early when another warp of the CTA has raised the abort flag.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < (1u << 24); ++i) {
    if (sm100::mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  return false;
}

__global__ void __launch_bounds__(TMA_THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            DecodeTcParams p, IertBatchView b, IertKvView c) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ int red[8];
  __shared__ __align__(8) uint64_t full_bar[NSTAGE], empty_bar[NSTAGE], prod_done;
  __shared__ volatile int abort_s, armed_s;      // a wait ran out; pages the producer has asked for
  // the swizzle pattern repeats every 1,024 bytes of shared memory: the ring starts on such a boundary
  uint8_t* smem = smem_raw + ((1024u - (sm100::smem_addr(smem_raw) & 1023u)) & 1023u);
  auto k_tile = [&](int i) { return smem + (size_t)(2 * i) * TMA_TILE_BYTES; };
  auto v_tile = [&](int i) { return smem + (size_t)(2 * i + 1) * TMA_TILE_BYTES; };
  uint8_t* q_tile = smem + 2 * NSTAGE * TMA_TILE_BYTES;                     // [16][ROW_BYTES]
  float* cs_tab = reinterpret_cast<float*>(q_tile + ROWS * ROW_BYTES);
  __nv_bfloat16* new_kv = reinterpret_cast<__nv_bfloat16*>(cs_tab + HD);

  pdl_launch_dependents();
  const int split = blockIdx.z, t = blockIdx.y;
  const int kvh = blockIdx.x / p.slices, slice = blockIdx.x % p.slices;
  const int group = p.heads / c.kv_heads;
  const int g0 = slice * p.gt;
  const int n_g = min(p.gt, group - g0);
  const int head0 = kvh * group + g0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const bool consumer = warp < WARPS;
  auto consumer_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); };

  const int s = sequence_of_token(b, t);
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  float* po = p.part_out + (((size_t)t * p.heads + head0) * p.splits + split) * HD;
  float* pml = p.part_ml + (((size_t)t * p.heads + head0) * p.splits + split) * 2;
  if (slot < 0) {
    pdl_wait();
    if (p.splits == 1) {
      for (int i = threadIdx.x; i < n_g * HD; i += TMA_THREADS)
        p.out[((size_t)t * p.heads + head0) * HD + i] = __float2bfloat16_rn(0.f);
    } else if (threadIdx.x < n_g) {
      pml[(size_t)threadIdx.x * p.splits * 2] = -INFINITY; pml[(size_t)threadIdx.x * p.splits * 2 + 1] = 0.f;
    }
    return;
  }
  const int pos = b.pos0[s] + (t - b.cu_q[s]);
  const int j_min = c.window > 0 ? max(0, pos + 1 - c.window) : 0;
  const int pg_lo = j_min / PAGE, pg_hi = pos / PAGE + 1;
  int n_splits = p.splits;
  if (p.target_ctas > 0 && p.splits > 1) {
    n_splits = balanced_parts(b, c, pg_hi - pg_lo, p.splits, p.target_ctas, gridDim.x, red);
    if (split >= n_splits) return;
  }
  const int per = (pg_hi - pg_lo + n_splits - 1) / n_splits;
  const int my_lo = pg_lo + split * per, my_hi = min(pg_hi, my_lo + per);
  const bool fused = p.rope && p.store;
  const bool own_new_row = fused && my_lo < my_hi && my_hi == pg_hi;
  const int half = p.rotary_dim / 2;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTAGE; ++i) { sm100::mbar_init(&full_bar[i], 1); sm100::mbar_init(&empty_bar[i], WARPS); }
    sm100::mbar_init(&prod_done, 1);
    abort_s = 0; armed_s = 0;
    sm100::mbar_fence_init();
  }
  __syncthreads();

  if (!consumer) {
    // ---- the producer: page numbers of up to 32 pages at a time, one per lane, then one thread
    // arms the barrier and asks for the boxes
    if (lane == 0) { sm100::tma_prefetch_desc(&map_k); sm100::tma_prefetch_desc(&map_v); }
    bool waited = false, stop = false;
    int armed = 0;
    for (int base = my_lo; base < my_hi; base += 32) {
      const int mine = base + lane;
      int page = -1;
      if (mine < my_hi) page = c.page_table[(size_t)slot * c.table_width + mine % c.ring_pages];
      for (int k = 0; k < 32 && base + k < my_hi; ++k) {
        const int pg = base + k, i = pg - my_lo, buf = i % NSTAGE;
        const int pgid = __shfl_sync(0xffffffffu, page, k);
        const bool ok = pgid >= 0 && pgid < c.n_pages;
        if (lane != 0 || stop) continue;
        if (abort_s) { stop = true; continue; }
        if (!ok) atomicOr(p.err, IERT_ERR_PAGE_RANGE);
        // without the fused cache write the kernel in front wrote the newest row: wait for it first
        if (!fused && !waited && pg == pos / PAGE) { pdl_wait(); waited = true; }
        if (i >= NSTAGE && !wait_or_abort(&empty_bar[buf], ((i / NSTAGE) - 1) & 1, &abort_s)) {
          // the slot may still be in use: nothing more is asked for
          if (!abort_s) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
          abort_s = 1;
          stop = true;
          continue;
        }
        sm100::mbar_expect_tx(&full_bar[buf], 2 * TMA_TILE_BYTES);
        const int row0 = ((ok ? pgid : 0) * c.kv_heads + kvh) * PAGE;
#pragma unroll
        for (int bx = 0; bx < BOXES; ++bx) {
          sm100::tma_load_2d(k_tile(buf) + bx * BOX_BYTES, &map_k, &full_bar[buf], bx * 64, row0);
          sm100::tma_load_2d(v_tile(buf) + bx * BOX_BYTES, &map_v, &full_bar[buf], bx * 64, row0);
        }
        armed = i + 1;
      }
    }
    if (lane == 0) {               // tell the consumers how far the producer came, and that it has stopped
      armed_s = armed;
      __threadfence_block();
      sm100::mbar_arrive(&prod_done);
    }
    return;
  }

  // ---- consumers
  if (p.rope) {
    for (int k = threadIdx.x; k < half; k += THREADS) {
      float sn, cs_;
      sincosf((float)pos * p.inv_freq[k], &sn, &cs_);
      cs_tab[k] = cs_;
      cs_tab[half + k] = sn;
    }
  }
  const __nv_bfloat16* tok_row = p.qkv + (size_t)t * ((size_t)(p.heads + 2 * c.kv_heads) * HD);
  auto rotate_into = [&](const __nv_bfloat16* src, __nv_bfloat16* dst, int k) {
    const int i0 = p.pairing == IERT_PAIR_HALF ? k : 2 * k;
    const int i1 = p.pairing == IERT_PAIR_HALF ? k + half : 2 * k + 1;
    const float a = __bfloat162float(src[i0]), bb = __bfloat162float(src[i1]);
    dst[i0] = __float2bfloat16_rn(a * cs_tab[k] - bb * cs_tab[half + k]);
    dst[i1] = __float2bfloat16_rn(a * cs_tab[half + k] + bb * cs_tab[k]);
  };
  pdl_wait();
  {
    const __nv_bfloat16* q = tok_row + (size_t)head0 * HD;
    if (p.rope) {
      consumer_sync();                                   // the angle table is complete
      for (int i = threadIdx.x; i < ROWS * (HD / 2); i += THREADS) {
        const int r = i / (HD / 2), k = i % (HD / 2);
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(q_tile + r * ROW_BYTES);
        if (r >= n_g) { dst[2 * k] = __float2bfloat16_rn(0.f); dst[2 * k + 1] = __float2bfloat16_rn(0.f); }
        else if (k < half) rotate_into(q + r * HD, dst, k);
        else { const int d = p.rotary_dim + 2 * (k - half); dst[d] = q[r * HD + d]; dst[d + 1] = q[r * HD + d + 1]; }
      }
    } else {
      constexpr int CHUNKS = HD / 8;
      for (int i = threadIdx.x; i < ROWS * CHUNKS; i += THREADS) {
        const int r = i / CHUNKS, cc = i % CHUNKS;
        const uint4 val = r < n_g ? *reinterpret_cast<const uint4*>(q + r * HD + cc * 8) : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(q_tile + r * ROW_BYTES + cc * 16) = val;
      }
    }
  }
  if (own_new_row) {
    const __nv_bfloat16* kn = tok_row + (size_t)(p.heads + kvh) * HD;
    const __nv_bfloat16* vn = tok_row + (size_t)(p.heads + c.kv_heads + kvh) * HD;
    for (int k = threadIdx.x; k < HD / 2; k += THREADS) {
      if (k < half) rotate_into(kn, new_kv, k);
      else { const int d = p.rotary_dim + 2 * (k - half); new_kv[d] = kn[d]; new_kv[d + 1] = kn[d + 1]; }
      new_kv[HD + 2 * k] = vn[2 * k];
      new_kv[HD + 2 * k + 1] = vn[2 * k + 1];
    }
  }
  consumer_sync();
  if (own_new_row && slice == 0) {
    const int page = c.page_table[(size_t)slot * c.table_width + (pos / PAGE) % c.ring_pages];
    if (page >= 0 && page < c.n_pages) {
      const size_t off = ((((size_t)page * c.kv_heads + kvh) * PAGE) + pos % PAGE) * HD;
      for (int d = threadIdx.x; d < HD; d += THREADS) {
        ((__nv_bfloat16*)c.k)[off + d] = new_kv[d];
        ((__nv_bfloat16*)c.v)[off + d] = new_kv[HD + d];
      }
    } else if (threadIdx.x == 0) {
      atomicOr(p.err, IERT_ERR_PAGE_RANGE);
    }
  }
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    ldsm4(qf[ks], q_tile + (lane & 15) * ROW_BYTES + (ks * 16 + (lane >> 4) * 8) * 2);
  float o[KSTEPS * 2][4];
#pragma unroll
  for (int n = 0; n < KSTEPS * 2; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_row = -INFINITY, l_row = 0.f;

  for (int pg = my_lo; pg < my_hi; ++pg) {
    const int i = pg - my_lo, buf = i % NSTAGE;
    if (!wait_or_abort(&full_bar[buf], (i / NSTAGE) & 1, &abort_s)) {
      if (lane == 0 && !abort_s) atomicOr(p.err, IERT_ERR_WAIT_EXPIRED);
      __syncwarp();
      abort_s = 1;
      break;
    }
    // this warp's 16 positions of the page: rows [16 warp, 16 warp + 16)
    const int row_lo = max(0, j_min - pg * PAGE);
    int row_hi = min(PAGE - 1, pos - pg * PAGE);
    const bool patch = own_new_row && pg == pos / PAGE;
    if (patch) --row_hi;                                      // the newest row comes from the projection
    const int w0 = warp * 16;
    bool wrote = false;
    if (row_lo > w0 || row_hi < w0 + 15) {                    // rows of the values that must not count
      for (int r = w0; r < w0 + 16; ++r) {
        if ((r >= row_lo && r <= row_hi) || (patch && r == pos % PAGE)) continue;      // (the patched row: below)
#pragma unroll
        for (int bx = 0; bx < BOXES; ++bx)
          reinterpret_cast<uint32_t*>(v_tile(buf) + bx * BOX_BYTES + r * 128)[lane] = 0u;
      }
      wrote = true;
    }
    if (patch && pos % PAGE >= w0 && pos % PAGE < w0 + 16) {
      const int r = pos % PAGE;
      for (int d = lane; d < HD; d += 32) {
        reinterpret_cast<__nv_bfloat16*>(swz(k_tile(buf), r, d & ~7))[d & 7] = new_kv[d];
        reinterpret_cast<__nv_bfloat16*>(swz(v_tile(buf), r, d & ~7))[d & 7] = new_kv[HD + d];
      }
      wrote = true;
    }
    if (wrote) __syncwarp();
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t kb[4];
      ldsm4(kb, swz(k_tile(buf), w0 + (lane & 7) + ((lane >> 4) << 3), ks * 16 + ((lane >> 3) & 1) * 8));
      mma16816(sc[0], qf[ks], kb[0], kb[1]);
      mma16816(sc[1], qf[ks], kb[2], kb[3]);
    }
    const int jbase = pg * PAGE + w0;
    float mx = m_row;
    float v[2][2];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = jbase + n * 8 + tq * 2 + e;
        v[n][e] = (j >= j_min && j <= pos) ? sc[n][e] * p.scale_log2e : -INFINITY;
        mx = fmaxf(mx, v[n][e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float alpha = m_row == -INFINITY ? 0.f : exp2f(m_row - mx);
    m_row = mx;
    l_row *= alpha;
    float pr[2][2];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[n][e] = (v[n][e] == -INFINITY || mx == -INFINITY) ? 0.f : exp2f(v[n][e] - mx);
        l_row += pr[n][e];
      }
#pragma unroll
    for (int n = 0; n < KSTEPS * 2; ++n) { o[n][0] *= alpha; o[n][1] *= alpha; }
    const uint32_t pa[4] = {pack2(pr[0][0], pr[0][1]), 0u, pack2(pr[1][0], pr[1][1]), 0u};
#pragma unroll
    for (int dp = 0; dp < KSTEPS; ++dp) {
      uint32_t vb[4];
      ldsm4t(vb, swz(v_tile(buf), w0 + (lane & 7) + (((lane >> 3) & 1) << 3), dp * 16 + (lane >> 4) * 8));
      mma16816(o[2 * dp], pa, vb[0], vb[1]);
      mma16816(o[2 * dp + 1], pa, vb[2], vb[3]);
    }
    if (wrote) sm100::fence_proxy_async_smem();          // the slot's next page arrives through the async proxy
    __syncwarp();
    if (lane == 0) sm100::mbar_arrive(&empty_bar[buf]);
  }

  // ---- merge the four warps in warp order (every page has been used: the ring is free)
  consumer_sync();
  if (abort_s) {                   // the same for all four warps: every write of the flag precedes the barrier
    // A wait ran out somewhere in this CTA.  Copies that the producer asked for may still be on
    // their way into the ring: wait (bounded) until the producer has stopped, then for the last
    // page asked for in every slot, before the ring is touched or the CTA leaves.
    if (threadIdx.x == 0) {
      sm100::mbar_wait(&prod_done, 0);
      const int armed = armed_s;
      for (int buf = 0; buf < NSTAGE; ++buf) {
        if (armed <= buf) continue;
        const int last = ((armed - 1 - buf) / NSTAGE) * NSTAGE + buf;      // the last page asked for in this slot
        sm100::mbar_wait(&full_bar[buf], (last / NSTAGE) & 1);
      }
    }
    consumer_sync();
    // no merge of what the warps hold: an empty partial result (the merge kernel skips it), or zeros
    if (p.splits == 1) {
      for (int i = threadIdx.x; i < n_g * HD; i += THREADS)
        p.out[((size_t)t * p.heads + head0) * HD + i] = __float2bfloat16_rn(0.f);
    } else if (threadIdx.x < n_g) {
      pml[(size_t)threadIdx.x * p.splits * 2] = -INFINITY; pml[(size_t)threadIdx.x * p.splits * 2 + 1] = 0.f;
    }
    return;
  }
  l_row += __shfl_xor_sync(0xffffffffu, l_row, 1);
  l_row += __shfl_xor_sync(0xffffffffu, l_row, 2);
  float* o_s = reinterpret_cast<float*>(smem);                 // [WARPS][8][HD]
  float* ml_s = o_s + WARPS * 8 * HD;                          // [WARPS][8][2]
#pragma unroll
  for (int n = 0; n < KSTEPS * 2; ++n) {
    o_s[(warp * 8 + g) * HD + n * 8 + tq * 2] = o[n][0];
    o_s[(warp * 8 + g) * HD + n * 8 + tq * 2 + 1] = o[n][1];
  }
  if (tq == 0) { ml_s[(warp * 8 + g) * 2] = m_row; ml_s[(warp * 8 + g) * 2 + 1] = l_row; }
  consumer_sync();
  const bool direct = p.splits == 1;
  for (int r = 0; r < n_g && r < 8; ++r) {
    float mm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, ml_s[(w * 8 + r) * 2]);
    float wgt[WARPS], ll = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      const float mw = ml_s[(w * 8 + r) * 2];
      wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      ll += wgt[w] * ml_s[(w * 8 + r) * 2 + 1];
    }
    const float inv = ll > 0.f ? 1.0f / ll : 0.f;
    for (int d = threadIdx.x; d < HD; d += THREADS) {
      float acc = 0.f;
      for (int w = 0; w < WARPS; ++w) acc += wgt[w] * o_s[(w * 8 + r) * HD + d];
      if (direct) p.out[((size_t)t * p.heads + head0 + r) * HD + d] = __float2bfloat16_rn(acc * inv);
      else po[(size_t)r * p.splits * HD + d] = acc;
    }
    if (!direct && threadIdx.x == 0) { pml[(size_t)r * p.splits * 2] = mm; pml[(size_t)r * p.splits * 2 + 1] = ll; }
  }
}
#endif  // HEAD_DIM % 64 == 0

// One block per (token, head): merge the splits in split order, normalise, write bf16.
__global__ void attention_decode_tc_combine_kernel(DecodeTcParams p, IertBatchView b, IertKvView c) {
  __shared__ int red[8];
  pdl_launch_dependents();     // the next kernel may start its preamble now
  const int t = blockIdx.x, head = blockIdx.y;
  // how many parts this token's sequence was cut into (the attention kernel computed the same)
  int n_splits = p.splits;
  const int s_ = sequence_of_token(b, t);
  const bool live = s_ >= 0 && b.slot_ids[s_] >= 0;
  if (p.target_ctas > 0 && p.splits > 1 && live) {
    const int pos = b.pos0[s_] + (t - b.cu_q[s_]);
    const int j_min = c.window > 0 ? max(0, pos + 1 - c.window) : 0;
    const int group = p.heads / c.kv_heads;
    n_splits = balanced_parts(b, c, pos / PAGE + 1 - j_min / PAGE, p.splits, p.target_ctas,
                              c.kv_heads * ((group + p.gt - 1) / p.gt), red);
  }
  pdl_wait();                  // everything below may depend on the kernel before
  __nv_bfloat16* o = p.out + ((size_t)t * p.heads + head) * HD;
  if (!live) {                 // a padding sequence: zeros
    for (int d = threadIdx.x; d < HD; d += blockDim.x) o[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const float* po = p.part_out + ((size_t)t * p.heads + head) * p.splits * HD;
  const float* pml = p.part_ml + ((size_t)t * p.heads + head) * p.splits * 2;
  float mm = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, pml[2 * s]);
  float ll = 0.f;
  for (int s = 0; s < n_splits; ++s) ll += pml[2 * s] == -INFINITY ? 0.f : exp2f(pml[2 * s] - mm) * pml[2 * s + 1];
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; ++s)
      if (pml[2 * s] != -INFINITY) acc += exp2f(pml[2 * s] - mm) * po[(size_t)s * HD + d];
    o[d] = __float2bfloat16_rn(acc * inv);
  }
}

}  // namespace

// CTAs of these kernels that one SM holds at once, as the callers' rules for cutting sequences
// into parts assume it: two (with 128-wide heads the three-page rings of keys and values take
// half an SM's shared memory; the TMA kernel's 160 threads x 168 registers allow two as well).
// Smaller heads would fit more, but the rules were measured with two.
IERT_API int iert_attention_decode_tc_ctas_per_sm() { return 2; }

IERT_API long long iert_attention_decode_tc_scratch_floats(int n_tokens, int heads, int splits) {
  return (long long)n_tokens * heads * splits * (HD + 2);
}

namespace {

int launch_decode(const void* qkv, void* out, const IertBatchView* batch, const IertKvView* cache, int heads,
                  float scale, int splits, int target_ctas, float* scratch, const float* inv_freq, int rope, int rotary_dim,
                  int pairing, int store, int* err, cudaStream_t stream) {
  const int T = batch->n_tokens;
  if (T <= 0) return IERT_OK;
  if (cache->dtype != IERT_BF16 || cache->head_dim != HD || cache->page_tokens != PAGE || splits < 1 || heads <= 0 ||
      cache->kv_heads <= 0 || heads % cache->kv_heads != 0 || T > 65535)
    return IERT_BAD_ARGUMENT;
  if (rope && (!inv_freq || rotary_dim < 0 || rotary_dim > HD || (rotary_dim & 1) ||
               (pairing != IERT_PAIR_HALF && pairing != IERT_PAIR_INTERLEAVED)))
    return IERT_BAD_ARGUMENT;
  const int group = heads / cache->kv_heads;
  DecodeTcParams p;
  p.qkv = (const __nv_bfloat16*)qkv;
  p.out = (__nv_bfloat16*)out;
  p.heads = heads; p.splits = splits; p.target_ctas = target_ctas > 0 ? target_ctas : 0;
  p.gt = group < 8 ? group : 8;                      // heads per CTA (rows 0..7 of the MMA tile)
  p.slices = (group + p.gt - 1) / p.gt;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.err = err;
  p.part_out = scratch;
  p.part_ml = scratch + (size_t)T * heads * splits * HD;
  p.inv_freq = inv_freq; p.rope = rope; p.rotary_dim = rotary_dim; p.pairing = pairing; p.store = store;
  if (splits > 65535) return IERT_BAD_ARGUMENT;
  // page ring, query tile, angle table and the step's own key/value row
  size_t smem = 2 * NSTAGE * (size_t)TILE_BYTES + ROWS * ROW_BYTES + 8 * (size_t)HD;
  const size_t merge = (size_t)(WARPS * 8 * HD + WARPS * 8 * 2) * sizeof(float);
  if (merge > smem) smem = merge;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return IERT_CUDA_ERROR;
    }
    configured = true;
  }
  bool launched = false;
#if HEAD_DIM % 64 == 0
  // pages by TMA where the head size allows (IERT_DECODE_TMA=0: the cp.async kernel, for comparison)
  static const bool use_tma = [] { const char* e = getenv("IERT_DECODE_TMA"); return !(e && e[0] == '0'); }();
  CUtensorMap map_k, map_v;
  const long long cache_rows = (long long)cache->n_pages * cache->kv_heads * PAGE;
  if (use_tma && tma_host::tensor_map_2d(cache->k, cache_rows, HD, HD, PAGE, &map_k) &&
      tma_host::tensor_map_2d(cache->v, cache_rows, HD, HD, PAGE, &map_v)) {
    const size_t ring = 2 * NSTAGE * (size_t)TMA_TILE_BYTES;
    size_t smem_tma = ring + ROWS * ROW_BYTES + 8 * (size_t)HD + 1024;      // (+ alignment of the ring)
    if (merge > ring) smem_tma += merge - ring;
    static bool configured_tma = false;
    if (!configured_tma) {
      if (cudaFuncSetAttribute(attention_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_tma) != cudaSuccess) {
        cudaGetLastError();
        return IERT_CUDA_ERROR;
      }
      configured_tma = true;
    }
    launch_dep(attention_decode_tma_kernel, dim3(cache->kv_heads * p.slices, T, splits), dim3(TMA_THREADS), smem_tma, stream,
               map_k, map_v, p, *batch, *cache);
    launched = true;
  }
#endif
  if (!launched)
    launch_dep(attention_decode_tc_kernel, dim3(cache->kv_heads * p.slices, T, splits), dim3(THREADS), smem, stream,
               p, *batch, *cache);
  if (cudaGetLastError() != cudaSuccess) return IERT_CUDA_ERROR;
  if (splits == 1) return IERT_OK;                   // nothing to merge: the kernel wrote the output
  launch_dep(attention_decode_tc_combine_kernel, dim3(T, heads), dim3(HD >= 128 ? 128 : 64), 0, stream, p, *batch, *cache);
  return cudaGetLastError() == cudaSuccess ? IERT_OK : IERT_CUDA_ERROR;
}

}  // namespace

// `splits`: the most parts a sequence's keys are cut into; with target_ctas > 0 each sequence is cut
// into as many of them as its length asks for (see balanced_parts), else every sequence into all.
// Same contract as the core library's iert_attention_decode, for caches with head_dim ==
// HEAD_DIM, bf16, 64-position pages.  Anything else: IERT_BAD_ARGUMENT, nothing launched.
IERT_API int iert_attention_decode_tc(const void* qkv, void* out, const IertBatchView* batch,
                                      const IertKvView* cache, int heads, float scale, int splits,
                                      int target_ctas, float* scratch, int* err, cudaStream_t stream) {
  return launch_decode(qkv, out, batch, cache, heads, scale, splits, target_ctas, scratch, nullptr, 0, 0, 0, 0, err,
                       stream);
}

// The same with the rotary encoding and the cache write of the step inside the kernel: `qkv` is
// the raw projection of one token per sequence and is left as it is; queries and the new key
// are rotated on the way (angles pos * inv_freq[k], pairs by `pairing`, the first `rotary_dim`
// dimensions of a head); with store != 0 the new key and value are written to the cache.
IERT_API int iert_attention_decode_tc_rope(const void* qkv, void* out, const IertBatchView* batch,
                                           const IertKvView* cache, int heads, float scale, int splits,
                                           int target_ctas, float* scratch, const float* inv_freq, int rotary_dim,
                                           int pairing, int store, int* err, cudaStream_t stream) {
  if (batch->n_tokens != batch->n_seqs) return IERT_BAD_ARGUMENT;     // one token per sequence
  return launch_decode(qkv, out, batch, cache, heads, scale, splits, target_ctas, scratch, inv_freq, 1, rotary_dim,
                       pairing, store, err, stream);
}
