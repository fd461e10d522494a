// Decode attention over the paged cache: one query token per sequence, split over the
// keys ("split-KV") so that a small batch still fills the GPU, then a combine pass.
//
//   grid (splits, kv_heads * slices, sequences); a CTA serves up to GT query heads that
//   share one kv head, so each key and value is read once for the whole group.
//   Keys are walked in blocks of 32 (never across a page).  Each of the 4 warps owns every
//   4th block of the CTA's key range and keeps its own running maximum / sum / output
//   (online softmax, fp32), merged through shared memory at the end.
//   Scores: lane = key, the dot product over head_dim runs inside the thread (16-byte loads
//   of the key row, the queries broadcast from shared memory).
//   Values: lane = a pair of dimensions (and +64, +128, +192 for larger heads); the block's
//   probabilities are broadcast from shared memory.
//   Partial results (unnormalised output, maximum, sum) of every split go to scratch memory;
//   `attention_decode_combine` merges them in split order and writes the bf16 output.
//
// Formulas as in the reference's decode path (src/layers/attention.rs:609-645): the visible
// keys are [max(0, total - W), total) with total = position + 1; scale 1/sqrt(head_dim)
// comes from the caller; softmax in fp32 (src/ops/softmax.rs:11-25).
#include "common.cuh"

using namespace iert;

namespace {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int KEY_BLOCK = 32;
constexpr int MAX_PAIR_ITERS = 4;            // head_dim <= 256

struct DecodeParams {
  const __nv_bfloat16* qkv;   // [T, (heads + 2 kv_heads) * hd], queries rotated
  float* part_out;            // [T, heads, splits, hd]
  float* part_ml;             // [T, heads, splits, 2]
  __nv_bfloat16* out;         // [T, heads * hd]
  int heads, splits, slices;
  float scale;
  int* err;
};

template <int GT>
__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(DecodeParams p, IertBatchView b, IertKvView c) {
  extern __shared__ float smem[];
  const int hd = c.head_dim;
  float* q_s = smem;                              // [GT][hd], pre-multiplied by the scale
  float* p_s = q_s + GT * hd;                     // [WARPS][KEY_BLOCK][GT]
  float* o_s = p_s + WARPS * KEY_BLOCK * GT;      // [WARPS][GT][hd]
  float* ml_s = o_s + WARPS * GT * hd;            // [WARPS][GT][2]

  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  const int split = blockIdx.x, t = blockIdx.z;
  const int kvh = blockIdx.y / p.slices, slice = blockIdx.y % p.slices;
  const int group = p.heads / c.kv_heads;
  const int g0 = slice * GT;                      // first head of the group this CTA serves
  const int n_g = min(GT, group - g0);
  const int head0 = kvh * group + g0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int s = b.tok_seq[t];
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  float* po = p.part_out + (((size_t)t * p.heads + head0) * p.splits + split) * hd;
  float* pml = p.part_ml + (((size_t)t * p.heads + head0) * p.splits + split) * 2;
  if (slot < 0) {                                 // padding: an empty partial
    for (int g = 0; g < n_g; ++g) {
      if (threadIdx.x == 0) { pml[(size_t)g * p.splits * 2] = -INFINITY; pml[(size_t)g * p.splits * 2 + 1] = 0.f; }
    }
    return;
  }
  const int pos = b.pos0[s] + (t - b.cu_q[s]);
  const int j_min = c.window > 0 ? max(0, pos + 1 - c.window) : 0;
  // the CTA's share of the 32-key blocks that hold [j_min, pos]
  const int blk_lo = j_min / KEY_BLOCK, blk_hi = pos / KEY_BLOCK + 1;
  const int per = (blk_hi - blk_lo + p.splits - 1) / p.splits;
  const int my_lo = blk_lo + split * per, my_hi = min(blk_hi, my_lo + per);

  const int row_elems = (p.heads + 2 * c.kv_heads) * hd;
  const __nv_bfloat16* q = p.qkv + (size_t)t * row_elems + (size_t)head0 * hd;
  for (int i = threadIdx.x; i < GT * hd; i += THREADS) {
    const int g = i / hd;
    q_s[i] = g < n_g ? __bfloat162float(q[i]) * p.scale : 0.f;
  }
  __syncthreads();

  float m[GT], l[GT], acc[GT][MAX_PAIR_ITERS][2];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PAIR_ITERS; ++i) acc[g][i][0] = acc[g][i][1] = 0.f;
  }
  float* p_w = p_s + warp * KEY_BLOCK * GT;
  const int pairs = hd / 2;
  const int blocks_per_page = c.page_tokens / KEY_BLOCK;

  for (int blk = my_lo + warp; blk < my_hi; blk += WARPS) {
    const int lblk = blk / blocks_per_page;                       // logical page of the sequence
    const int page = c.page_table[(size_t)slot * c.table_width + lblk % c.ring_pages];
    if (page < 0 || page >= c.n_pages) {
      if (lane == 0) atomicOr(p.err, IERT_ERR_PAGE_RANGE);
      continue;
    }
    const size_t page_off = (((size_t)page * c.kv_heads + kvh) * c.page_tokens +
                             (size_t)(blk % blocks_per_page) * KEY_BLOCK) * hd;
    const int j = blk * KEY_BLOCK + lane;
    const bool visible = j >= j_min && j <= pos;

    // ---- scores: this lane's key against the group's queries
    float sc[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) sc[g] = 0.f;
    if (visible) {
      const uint4* krow = reinterpret_cast<const uint4*>((const __nv_bfloat16*)c.k + page_off + (size_t)lane * hd);
      const int n8 = hd / 8;
      for (int d8 = 0; d8 < n8; d8 += 4) {             // four 16-byte loads in flight per thread
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) raw[u] = d8 + u < n8 ? krow[d8 + u] : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (d8 + u >= n8) break;
          const __nv_bfloat162* kk = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
          float kf[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(kk[e]);
            kf[2 * e] = f.x; kf[2 * e + 1] = f.y;
          }
#pragma unroll
          for (int g = 0; g < GT; ++g) {
            const float4 qa = *reinterpret_cast<const float4*>(q_s + g * hd + (d8 + u) * 8);
            const float4 qb = *reinterpret_cast<const float4*>(q_s + g * hd + (d8 + u) * 8 + 4);
            sc[g] = fmaf(qa.x, kf[0], sc[g]); sc[g] = fmaf(qa.y, kf[1], sc[g]);
            sc[g] = fmaf(qa.z, kf[2], sc[g]); sc[g] = fmaf(qa.w, kf[3], sc[g]);
            sc[g] = fmaf(qb.x, kf[4], sc[g]); sc[g] = fmaf(qb.y, kf[5], sc[g]);
            sc[g] = fmaf(qb.z, kf[6], sc[g]); sc[g] = fmaf(qb.w, kf[7], sc[g]);
          }
        }
      }
    }
    // ---- online softmax over the block
    float alpha[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float v = visible ? sc[g] : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(v));
      const float pj = visible ? __expf(v - m_new) : 0.f;
      alpha[g] = m[g] == -INFINITY ? 0.f : __expf(m[g] - m_new);
      l[g] = l[g] * alpha[g] + pj;                 // per-lane share of the sum; reduced at the end
      m[g] = m_new;
      p_w[lane * GT + g] = pj;
    }
    __syncwarp();
    // ---- values: this lane's dimensions over the block's keys
    // only rows of visible keys are read: a row outside [j_min, pos] may never have been written
    const int n_keys = min(KEY_BLOCK, pos - blk * KEY_BLOCK + 1);
    const int jj_lo = max(0, j_min - blk * KEY_BLOCK);
    const __nv_bfloat162* vbase = reinterpret_cast<const __nv_bfloat162*>((const __nv_bfloat16*)c.v + page_off);
#pragma unroll
    for (int i = 0; i < MAX_PAIR_ITERS; ++i) {
      const int pr = lane + 32 * i;
      if (pr >= pairs) break;
#pragma unroll
      for (int g = 0; g < GT; ++g) { acc[g][i][0] *= alpha[g]; acc[g][i][1] *= alpha[g]; }
      for (int jj = jj_lo; jj < n_keys; jj += 8) {     // eight value rows in flight per thread
        __nv_bfloat162 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          raw[u] = jj + u < n_keys ? vbase[(size_t)(jj + u) * pairs + pr] : __nv_bfloat162();
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (jj + u >= n_keys) break;
          const float2 vv = __bfloat1622float2(raw[u]);
#pragma unroll
          for (int g = 0; g < GT; ++g) {
            const float pj = p_w[(jj + u) * GT + g];
            acc[g][i][0] = fmaf(pj, vv.x, acc[g][i][0]);
            acc[g][i][1] = fmaf(pj, vv.y, acc[g][i][1]);
          }
        }
      }
    }
    __syncwarp();
  }

  // ---- merge the four warps (fixed order), write the split's partial
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    l[g] = warp_sum(l[g]);
    if (lane == 0) { ml_s[(warp * GT + g) * 2] = m[g]; ml_s[(warp * GT + g) * 2 + 1] = l[g]; }
#pragma unroll
    for (int i = 0; i < MAX_PAIR_ITERS; ++i) {
      const int pr = lane + 32 * i;
      if (pr < pairs) {
        o_s[(warp * GT + g) * hd + 2 * pr] = acc[g][i][0];
        o_s[(warp * GT + g) * hd + 2 * pr + 1] = acc[g][i][1];
      }
    }
  }
  __syncthreads();
  for (int g = 0; g < n_g; ++g) {
    float mm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, ml_s[(w * GT + g) * 2]);
    float wgt[WARPS], ll = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      const float mw = ml_s[(w * GT + g) * 2];
      wgt[w] = mw == -INFINITY ? 0.f : __expf(mw - mm);
      ll += wgt[w] * ml_s[(w * GT + g) * 2 + 1];
    }
    for (int d = threadIdx.x; d < hd; d += THREADS) {
      float o = 0.f;
      for (int w = 0; w < WARPS; ++w) o += wgt[w] * o_s[(w * GT + g) * hd + d];
      po[(size_t)g * p.splits * hd + d] = o;
    }
    if (threadIdx.x == 0) { pml[(size_t)g * p.splits * 2] = mm; pml[(size_t)g * p.splits * 2 + 1] = ll; }
  }
}

// One block per (token, head): merge the splits in split order, normalise, write bf16.
__global__ void attention_decode_combine_kernel(DecodeParams p, int hd) {
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  const int t = blockIdx.x, head = blockIdx.y;
  const float* po = p.part_out + ((size_t)t * p.heads + head) * p.splits * hd;
  const float* pml = p.part_ml + ((size_t)t * p.heads + head) * p.splits * 2;
  float mm = -INFINITY;
  for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, pml[2 * s]);
  float ll = 0.f;
  for (int s = 0; s < p.splits; ++s) ll += pml[2 * s] == -INFINITY ? 0.f : __expf(pml[2 * s] - mm) * pml[2 * s + 1];
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
  __nv_bfloat16* o = p.out + ((size_t)t * p.heads + head) * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.splits; ++s)
      if (pml[2 * s] != -INFINITY) acc += __expf(pml[2 * s] - mm) * po[(size_t)s * hd + d];
    o[d] = __float2bfloat16_rn(acc * inv);
  }
}

size_t smem_bytes(int gt, int hd) {
  return (size_t)(gt * hd + WARPS * KEY_BLOCK * gt + WARPS * gt * hd + WARPS * gt * 2) * sizeof(float);
}

}  // namespace

// Scratch the caller provides for `n_tokens` query tokens: floats for the partial outputs
// and for the (maximum, sum) pairs.
IERT_API long long iert_attention_decode_scratch_floats(int n_tokens, int heads, int head_dim, int splits) {
  return (long long)n_tokens * heads * splits * (head_dim + 2);
}

// qkv: packed bf16 projection of the step (one token per sequence), queries rotated, the new
// keys and values already stored in the cache.  out: bf16 [T, heads * head_dim].
// scratch: iert_attention_decode_scratch_floats(...) floats.  splits >= 1.
// Takes bf16 caches with head_dim a multiple of 8 up to 256 and page_tokens a multiple of 32;
// anything else returns IERT_BAD_ARGUMENT and launches nothing.
IERT_API int iert_attention_decode(const void* qkv, void* out, const IertBatchView* batch,
                                   const IertKvView* cache, int heads, float scale, int splits,
                                   float* scratch, int* err, cudaStream_t stream) {
  const int T = batch->n_tokens, hd = cache->head_dim;
  if (T <= 0) return IERT_OK;
  if (cache->dtype != IERT_BF16 || hd <= 0 || (hd & 7) || hd > 64 * MAX_PAIR_ITERS || splits < 1 ||
      cache->page_tokens % KEY_BLOCK != 0 || heads <= 0 || cache->kv_heads <= 0 || heads % cache->kv_heads != 0 ||
      T > 65535)
    return IERT_BAD_ARGUMENT;
  const int group = heads / cache->kv_heads;
  const int gt = group >= 8 ? 8 : group > 2 ? 4 : group;      // 1, 2, 4 or 8 heads per CTA
  DecodeParams p;
  p.qkv = (const __nv_bfloat16*)qkv;
  p.out = (__nv_bfloat16*)out;
  p.heads = heads; p.splits = splits; p.slices = (group + gt - 1) / gt;
  p.scale = scale; p.err = err;
  p.part_out = scratch;
  p.part_ml = scratch + (size_t)T * heads * splits * hd;
  if ((long long)cache->kv_heads * p.slices > 65535) return IERT_BAD_ARGUMENT;
  dim3 grid(splits, cache->kv_heads * p.slices, T);
  const size_t smem = smem_bytes(gt, hd);
  if (smem > 48 * 1024) return IERT_BAD_ARGUMENT;
  switch (gt) {
    case 1: launch_dep(attention_decode_kernel<1>, grid, THREADS, smem, stream, p, *batch, *cache); break;
    case 2: launch_dep(attention_decode_kernel<2>, grid, THREADS, smem, stream, p, *batch, *cache); break;
    case 4: launch_dep(attention_decode_kernel<4>, grid, THREADS, smem, stream, p, *batch, *cache); break;
    default: launch_dep(attention_decode_kernel<8>, grid, THREADS, smem, stream, p, *batch, *cache); break;
  }
  int st = iert_check_launch("attention_decode");
  if (st != IERT_OK) return st;
  launch_dep(attention_decode_combine_kernel, dim3(T, heads), dim3(hd >= 128 ? 128 : 64), 0, stream, p, hd);
  return iert_check_launch("attention_decode_combine");
}

// ---------------------------------------------------------------------------------------
// The variant that allocates nothing: see attention_decode_static.h for who needs it and
// for the rules.  The scratch lives in this translation unit's image.
#include "attention_decode_static.h"

#include <mutex>

namespace {

static __device__ __align__(256) float g_static_scratch[IERT_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_static_scratch_addr[MAX_DEVICES] = {};   // device address of the array, per device
std::mutex g_static_mu;

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the
// address a kernel can use has to be asked for, once per device, with that device current.
int static_scratch_address(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return IERT_STATIC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) {
      cudaGetLastError();
      return IERT_STATIC_SETUP_FAILED;
    }
    g_static_scratch_addr[dev] = (float*)p;
  }
  *out = g_static_scratch_addr[dev];
  return IERT_OK;
}

}  // namespace

IERT_API long long iert_attention_decode_static_capacity() { return (long long)IERT_STATIC_SCRATCH_FLOATS; }

IERT_API const char* iert_attention_decode_static_message(int status) {
  switch (status) {
    case IERT_OK: return "launched";
    case IERT_BAD_ARGUMENT: return "the kernel does not take this cache geometry or these sizes";
    case IERT_CUDA_ERROR: return "the launch failed (see iert_last_cuda_error)";
    case IERT_STATIC_SCRATCH_TOO_SMALL:
      return "the call needs more scratch than the library's fixed 8 MiB array holds: use fewer splits, a "
             "smaller batch, or iert_attention_decode with a buffer of your own";
    case IERT_STATIC_SETUP_FAILED: return "the device address of the fixed scratch array could not be obtained";
    default: return "unknown status";
  }
}

IERT_API int iert_attention_decode_static(const void* qkv, void* out, const IertBatchView* batch,
                                          const IertKvView* cache, int heads, float scale, int splits,
                                          int* err, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (splits < 1 || heads <= 0 || cache->head_dim <= 0) return IERT_BAD_ARGUMENT;
  const long long need = iert_attention_decode_scratch_floats(batch->n_tokens, heads, cache->head_dim, splits);
  if (need > (long long)IERT_STATIC_SCRATCH_FLOATS) return IERT_STATIC_SCRATCH_TOO_SMALL;
  float* scratch = nullptr;
  const int st = static_scratch_address(&scratch);
  if (st != IERT_OK) return st;
  return iert_attention_decode(qkv, out, batch, cache, heads, scale, splits, scratch, err, stream);
}
