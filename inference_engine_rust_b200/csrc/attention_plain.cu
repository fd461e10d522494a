// Plain attention on CUDA cores, all arithmetic in fp32: the true 32-bit path of the
// mixer for prompts and for decoding, and the reference sibling of the fast kernels.
// One block per (query token, head).  Keys are visited in chunks of the block size with a
// running maximum and sum, so the memory it needs does not grow with the context.
//
//   scores  s_j = (q . k_j) * scale for j in [j_min, pos], causal by construction
//   window  j_min = pos - (W - 1) (the last W keys, the current one included)
//   weights softmax over the visible keys; output = sum_j p_j v_j
// Reference: src/layers/attention.rs:364-415 (prompt), :609-645 (decode),
// src/ops/softmax.rs:11-25; grouped heads: kv_head = head / (heads / kv_heads), :243,372.
//
// Keys and values come either from the step's own packed projection ("fresh": a prompt
// that starts at position 0) or from the paged cache (decoding, or any step whose keys
// are all cached).
#include "common.cuh"

using namespace iert;

namespace {

constexpr int THREADS = 128;
constexpr int MAX_DIMS_PER_THREAD = 4;      // head_dim up to 512

template <typename T, bool PAGED>
__global__ void __launch_bounds__(THREADS)
attention_plain_kernel(const T* __restrict__ qkv, T* __restrict__ out, IertBatchView b,
                       IertKvView c, int heads, float scale, int* __restrict__ err) {
  extern __shared__ float smem[];
  const int hd = c.head_dim, nkv = c.kv_heads;
  float* q_s = smem;                  // [hd]
  float* p_s = smem + hd;             // [THREADS]
  float* scratch = p_s + THREADS;     // [33]

  const int t = blockIdx.x, head = blockIdx.y;
  const int row_elems = (heads + 2 * nkv) * hd;
  T* o = out + ((size_t)t * heads + head) * hd;
  const int s = b.tok_seq[t];
  const int slot = s >= 0 ? b.slot_ids[s] : -1;
  if (slot < 0) {                     // padding: defined output, nothing read
    for (int d = threadIdx.x; d < hd; d += THREADS) o[d] = from_f32<T>(0.f);
    return;
  }
  const int q_begin = b.cu_q[s];
  const int pos0 = b.pos0[s];
  const int pos = pos0 + (t - q_begin);
  const int j_min = c.window > 0 ? max(0, pos - (c.window - 1)) : 0;
  const int kvh = head / (heads / nkv);

  const T* q = qkv + (size_t)t * row_elems + (size_t)head * hd;
  for (int d = threadIdx.x; d < hd; d += THREADS) q_s[d] = to_f32(q[d]);
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[MAX_DIMS_PER_THREAD];
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_THREAD; ++i) acc[i] = 0.f;

  for (int j0 = j_min; j0 <= pos; j0 += THREADS) {
    const int j = j0 + threadIdx.x;
    float sc = -INFINITY;
    if (j <= pos) {
      const T* k;
      if (PAGED) {
        const long long off = kv_row_offset(c, slot, j, kvh, err);
        k = off >= 0 ? (const T*)c.k + off : nullptr;
      } else {
        k = qkv + (size_t)(q_begin + (j - pos0)) * row_elems + (size_t)(heads + kvh) * hd;
      }
      if (k) {
        float dot = 0.f;
        for (int d = 0; d < hd; ++d) dot = fmaf(q_s[d], to_f32(k[d]), dot);
        sc = dot * scale;
      }
    }
    const float m_new = fmaxf(m, block_max(sc, scratch));
    const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
    const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
    const float chunk_sum = block_sum(p, scratch);
    l = l * alpha + chunk_sum;
    m = m_new;
    p_s[threadIdx.x] = p;
    __syncthreads();
    const int n_in_chunk = min(THREADS, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_THREAD; ++i) {
      const int d = threadIdx.x + i * THREADS;
      if (d >= hd) break;
      float a = acc[i] * alpha;
      for (int jj = 0; jj < n_in_chunk; ++jj) {
        const float pj = p_s[jj];
        if (pj == 0.f) continue;
        const T* v;
        if (PAGED) {
          const long long off = kv_row_offset(c, slot, j0 + jj, kvh, nullptr);
          if (off < 0) continue;
          v = (const T*)c.v + off;
        } else {
          v = qkv + (size_t)(q_begin + (j0 + jj - pos0)) * row_elems + (size_t)(heads + nkv + kvh) * hd;
        }
        a = fmaf(pj, to_f32(v[d]), a);
      }
      acc[i] = a;
    }
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_THREAD; ++i) {
    const int d = threadIdx.x + i * THREADS;
    if (d < hd) o[d] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace

// qkv: packed [T, (heads + 2*kv_heads) * head_dim] projection, queries already rotated.
// out: [T, heads * head_dim].  paged = 0 reads keys/values from qkv (every sequence of the
// step must start at position 0); paged = 1 reads them from the cache view.
IERT_API int iert_attention_plain(const void* qkv, void* out, int dtype, const IertBatchView* batch,
                                  const IertKvView* cache, int heads, float scale, int paged,
                                  int* err, cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  const int hd = cache->head_dim;
  if (hd <= 0 || hd > THREADS * MAX_DIMS_PER_THREAD || heads <= 0 || cache->kv_heads <= 0 ||
      heads % cache->kv_heads != 0 || heads > 65535)
    return IERT_BAD_ARGUMENT;
  if (paged && cache->dtype != dtype) return IERT_BAD_ARGUMENT;
  dim3 grid(batch->n_tokens, heads);
  const size_t smem = (size_t)(hd + THREADS + 33) * sizeof(float);
#define GO(T, P) attention_plain_kernel<T, P><<<grid, THREADS, smem, stream>>>( \
    (const T*)qkv, (T*)out, *batch, *cache, heads, scale, err)
  if (dtype == IERT_F32) { if (paged) GO(float, true); else GO(float, false); }
  else if (dtype == IERT_BF16) { if (paged) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false); }
  else return IERT_BAD_ARGUMENT;
#undef GO
  return iert_check_launch("attention_plain");
}
