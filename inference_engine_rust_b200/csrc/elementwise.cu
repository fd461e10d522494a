// Memory-bound kernels of the step: embedding gather, RMSNorm (with optional row gather),
// rotary encoding fused with the cache write, SiLU(gate)*up, residual add, and the
// sequence-length update.  Statistics, angles and the residual stream are fp32 whatever
// the storage type.
#include "common.cuh"

using namespace iert;

// ---------------------------------------------------------------------------------------
// Embedding gather: x[t, :] = table[ids[t], :] * scale, x in fp32 (the residual stream).
// Reference: src/layers/embeddings.rs:15-17,119-139; scale src/engine/embed.rs:140-149.
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ x, int hidden, int vocab, float scale,
                                    int* __restrict__ err, IertNormAhead ahead) {
  __shared__ float scratch[33];
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  const int t = blockIdx.x;
  const int id = ids[t];
  float* row = x + (size_t)t * hidden;
  const bool in_range = id >= 0 && id < vocab;
  if (!in_range && threadIdx.x == 0) atomicOr(err, IERT_ERR_TOKEN_RANGE);
  const TW* src = table + (size_t)(in_range ? id : 0) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = in_range ? to_f32(src[i]) * scale : 0.f;
    row[i] = v;
    if (ahead.scaled_out) {    // the first half of the norm that follows (see IertNormAhead)
      const float g = ahead.weight_dtype == IERT_F32 ? ((const float*)ahead.weight)[i]
                                                     : __bfloat162float(((const __nv_bfloat16*)ahead.weight)[i]);
      ((__nv_bfloat16*)ahead.scaled_out)[(size_t)t * ahead.ld + i] = __float2bfloat16_rn(v * g);
      ss += v * v;
    }
  }
  if (ahead.scaled_out) {      // (the same for the whole block)
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) ahead.sumsq_out[t] = ss;
  }
}

// ahead (optional): the first half of the RMSNorm that follows, over the rows just written; ahead->parts is
// set to 1 (one sum of squares per row).
IERT_API int iert_embed_gather(const void* table, int table_dtype, const int* ids, float* x,
                               int n_tokens, int hidden, int vocab, float scale, int* err,
                               IertNormAhead* ahead, cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (hidden <= 0 || vocab <= 0) return IERT_BAD_ARGUMENT;
  IertNormAhead a = {nullptr, 0, nullptr, 0, nullptr, 0};
  if (ahead) {
    if (!ahead->weight || !ahead->scaled_out || !ahead->sumsq_out ||
        (ahead->weight_dtype != IERT_F32 && ahead->weight_dtype != IERT_BF16))
      return IERT_BAD_ARGUMENT;
    ahead->parts = 1;
    a = *ahead;
  }
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == IERT_F32)
    launch_dep(embed_gather_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, ids, x, hidden, vocab, scale, err, a);
  else if (table_dtype == IERT_BF16)
    launch_dep(embed_gather_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, x, hidden, vocab, scale, err, a);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("embed_gather");
}

// ---------------------------------------------------------------------------------------
// RMSNorm: out[r, i] = x[row(r), i] * w[i] / sqrt(mean(x^2) + eps), statistics in fp32.
// `rows_idx` (optional) gathers rows of x: the final norm runs only on the rows whose
// logits are wanted.  Reference: src/ops/rmsnorm.rs:38-48.
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                               TO* __restrict__ out, const int* __restrict__ rows_idx,
                               int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  const int r = blockIdx.x;
  const int src_row = rows_idx ? rows_idx[r] : r;
  const float* xr = x + (size_t)src_row * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = xr[i];
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rinv = 1.0f / sqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f32<TO>(xr[i] * to_f32(w[i]) * rinv);
}

// The same with the row held in registers (one read of x) and the scale vector fetched
// before the wait on the previous kernel, which it never depends on.
template <typename TW, typename TO, int NPT>
__global__ void rmsnorm_reg_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                                   TO* __restrict__ out, const int* __restrict__ rows_idx,
                                   int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();     // the next kernel may start its preamble now
  float wv[NPT], xv[NPT];
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    wv[k] = i < hidden ? to_f32(w[i]) : 0.f;
  }
  pdl_wait();                  // everything below may depend on the kernel before
  const int r = blockIdx.x;
  const int src_row = rows_idx ? rows_idx[r] : r;
  const float* xr = x + (size_t)src_row * hidden;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    xv[k] = i < hidden ? xr[i] : 0.f;
    ss += xv[k] * xv[k];
  }
  ss = block_sum(ss, scratch);
  const float rinv = 1.0f / sqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)r * hidden;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < hidden) o[i] = from_f32<TO>(xv[k] * wv[k] * rinv);
  }
}

// The same again with 16-byte accesses: a thread holds V runs of four consecutive elements.
// `hidden` a multiple of 4, all three pointers aligned for vectors of four.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TW, typename TO, int V>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                                   TO* __restrict__ out, const int* __restrict__ rows_idx,
                                   int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();     // the next kernel may start its preamble now
  const int n4 = hidden >> 2;
  float4 wv[V], xv[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int i4 = threadIdx.x + k * blockDim.x;
    wv[k] = i4 < n4 ? load4(w + 4 * i4) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();                  // everything below may depend on the kernel before
  const int r = blockIdx.x;
  const int src_row = rows_idx ? rows_idx[r] : r;
  const float* xr = x + (size_t)src_row * hidden;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int i4 = threadIdx.x + k * blockDim.x;
    xv[k] = i4 < n4 ? load4(xr + 4 * i4) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += xv[k].x * xv[k].x + xv[k].y * xv[k].y + xv[k].z * xv[k].z + xv[k].w * xv[k].w;
  }
  ss = block_sum(ss, scratch);
  const float rinv = 1.0f / sqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)r * hidden;
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int i4 = threadIdx.x + k * blockDim.x;
    if (i4 < n4)
      store4(o + 4 * i4, make_float4(xv[k].x * wv[k].x * rinv, xv[k].y * wv[k].y * rinv,
                                     xv[k].z * wv[k].z * rinv, xv[k].w * wv[k].w * rinv));
  }
}

IERT_API int iert_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype,
                          const int* rows_idx, int rows, int hidden, float eps,
                          cudaStream_t stream) {
  if (rows <= 0) return IERT_OK;
  if (hidden <= 0) return IERT_BAD_ARGUMENT;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const bool vec = (hidden & 3) == 0 && hidden <= 16 * 512 && (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
  const int n4 = hidden >> 2;
#define LAUNCH(TW, TO)                                                                                   \
  do {                                                                                                   \
    if (vec && n4 <= 128) launch_dep(rmsnorm_vec_kernel<TW, TO, 1>, rows, 128, 0, stream,                \
                                     x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);                  \
    else if (vec && n4 <= 512) launch_dep(rmsnorm_vec_kernel<TW, TO, 2>, rows, 256, 0, stream,           \
                                          x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);             \
    else if (vec && n4 <= 1024) launch_dep(rmsnorm_vec_kernel<TW, TO, 4>, rows, 256, 0, stream,          \
                                           x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);            \
    else if (vec) launch_dep(rmsnorm_vec_kernel<TW, TO, 4>, rows, 512, 0, stream,                        \
                             x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);                          \
    else if (hidden <= 4 * 256) launch_dep(rmsnorm_reg_kernel<TW, TO, 4>, rows, 256, 0, stream,               \
                                      x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);                 \
    else if (hidden <= 8 * 512) launch_dep(rmsnorm_reg_kernel<TW, TO, 8>, rows, 512, 0, stream,          \
                                           x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);            \
    else if (hidden <= 16 * 512) launch_dep(rmsnorm_reg_kernel<TW, TO, 16>, rows, 512, 0, stream,        \
                                             x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);          \
    else launch_dep(rmsnorm_kernel<TW, TO>, rows, threads, 0, stream,                                    \
                    x, (const TW*)w, (TO*)out, rows_idx, hidden, eps);                                   \
  } while (0)
  if (w_dtype == IERT_F32 && out_dtype == IERT_F32) LAUNCH(float, float);
  else if (w_dtype == IERT_F32 && out_dtype == IERT_BF16) LAUNCH(float, __nv_bfloat16);
  else if (w_dtype == IERT_BF16 && out_dtype == IERT_F32) LAUNCH(__nv_bfloat16, float);
  else if (w_dtype == IERT_BF16 && out_dtype == IERT_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return IERT_BAD_ARGUMENT;
#undef LAUNCH
  return iert_check_launch("rmsnorm");
}

// ---------------------------------------------------------------------------------------
// Rotary encoding of the query and key heads of a packed [T, (heads + 2*kv_heads)*head_dim]
// projection, in place, fused with the write of the rotated keys and the values into the
// paged cache.  A block serves one token and a run of its heads (all of them when the step
// has many tokens); heads [0, heads) are queries, the next kv_heads are keys, the last
// kv_heads are values.  The token's cos/sin table is computed once per block.
//   angle(pos, k) = pos * inv_freq[k] in fp32; (a, b) -> (a cos - b sin, a sin + b cos)
// Reference: src/ops/rope.rs:40-57 (rotation), src/layers/attention.rs:314-352 (order:
// rotate, then append), :518-520 (decode position = cache length before the append).
// A key or value is stored only if it can still be seen after this step: its position is
// within the last ring_pages*page_tokens positions of its sequence.
template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ qkv, IertBatchView b, IertKvView c,
                                     const float* __restrict__ inv_freq, int heads,
                                     int rotary_dim, int pairing, int write_cache,
                                     int heads_per_block, int vec8, int* __restrict__ err) {
  extern __shared__ float cs[];                 // [rotary_dim / 2] cos, then [rotary_dim / 2] sin
  pdl_launch_dependents();     // the next kernel may start its preamble now
  const int t = blockIdx.x;
  const int hd = c.head_dim, nkv = c.kv_heads;
  const int half = rotary_dim / 2;
  const int total_heads = heads + 2 * nkv;
  // The step's description (sequence, slot, position) and the angles do not depend on the
  // kernel before this one, only the projection does: everything up to the first read of
  // `qkv` runs while that kernel finishes.
  const int s = sequence_of_token(b, t);
  const int slot = s < 0 ? -1 : b.slot_ids[s];
  if (slot < 0) return;
  const int q_begin = b.cu_q[s], q_len = b.cu_q[s + 1] - q_begin;
  const int pos = b.pos0[s] + (t - q_begin);
  const int final_len = b.pos0[s] + q_len;
  for (int k = threadIdx.x; k < half; k += blockDim.x) {   // the token's angles, once for all heads
    float sn, cs_;
    sincosf((float)pos * inv_freq[k], &sn, &cs_);
    cs[k] = cs_;
    cs[half + k] = sn;
  }
  __syncthreads();
  pdl_wait();                  // the projection is complete from here on
  const bool store = write_cache && pos >= final_len - c.ring_pages * c.page_tokens;
  T* row = qkv + (size_t)t * total_heads * hd;
  // this block's heads: [h0, h1) of [queries | keys | values]
  const int h0 = blockIdx.y * heads_per_block, h1 = min(total_heads, h0 + heads_per_block);
  const int rot_end = min(h1, heads + nkv);            // heads below this index are rotated
  const int kv0 = max(h0, heads);                       // this block's key and value heads
  if (vec8) {
    // bf16 with 16-byte accesses: eight consecutive elements per thread and step
    __nv_bfloat16* rowb = reinterpret_cast<__nv_bfloat16*>(row);
    if (pairing == IERT_PAIR_HALF) {
      const int chunks = half / 8;
      for (int i = threadIdx.x; i < (rot_end - h0) * chunks; i += blockDim.x) {
        const int head = h0 + i / chunks, k0 = (i % chunks) * 8;
        __nv_bfloat16* vec = rowb + (size_t)head * hd;
        uint4 ra = *reinterpret_cast<const uint4*>(vec + k0), rb = *reinterpret_cast<const uint4*>(vec + half + k0);
        __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&ra);
        __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __bfloat1622float2(pa[e]), bb = __bfloat1622float2(pb[e]);
          const int k = k0 + 2 * e;
          pa[e] = __floats2bfloat162_rn(a.x * cs[k] - bb.x * cs[half + k], a.y * cs[k + 1] - bb.y * cs[half + k + 1]);
          pb[e] = __floats2bfloat162_rn(a.x * cs[half + k] + bb.x * cs[k], a.y * cs[half + k + 1] + bb.y * cs[k + 1]);
        }
        *reinterpret_cast<uint4*>(vec + k0) = ra;
        *reinterpret_cast<uint4*>(vec + half + k0) = rb;
      }
    } else {
      const int chunks = rotary_dim / 8;
      for (int i = threadIdx.x; i < (rot_end - h0) * chunks; i += blockDim.x) {
        const int head = h0 + i / chunks, c0 = (i % chunks) * 8;
        __nv_bfloat16* vec = rowb + (size_t)head * hd;
        uint4 rv = *reinterpret_cast<const uint4*>(vec + c0);
        __nv_bfloat162* pv = reinterpret_cast<__nv_bfloat162*>(&rv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 ab = __bfloat1622float2(pv[e]);
          const int k = c0 / 2 + e;
          pv[e] = __floats2bfloat162_rn(ab.x * cs[k] - ab.y * cs[half + k], ab.x * cs[half + k] + ab.y * cs[k]);
        }
        *reinterpret_cast<uint4*>(vec + c0) = rv;
      }
    }
    if (!store || kv0 >= h1) return;
    __syncthreads();                                    // the rotated keys are read back below
    const int chunks = hd / 8;
    for (int i = threadIdx.x; i < (h1 - kv0) * chunks; i += blockDim.x) {
      const int hh = kv0 + i / chunks - heads, d = (i % chunks) * 8;
      const bool is_k = hh < nkv;
      const long long off = kv_row_offset(c, slot, pos, is_k ? hh : hh - nkv, err);
      if (off < 0) continue;
      *reinterpret_cast<uint4*>((__nv_bfloat16*)(is_k ? c.k : c.v) + off + d) =
          *reinterpret_cast<const uint4*>(rowb + (size_t)(heads + hh) * hd + d);
    }
    return;
  }
  for (int i = threadIdx.x; i < (rot_end - h0) * half; i += blockDim.x) {
    const int head = h0 + i / half, k = i % half;
    const int i0 = pairing == IERT_PAIR_HALF ? k : 2 * k;
    const int i1 = pairing == IERT_PAIR_HALF ? k + half : 2 * k + 1;
    T* vec = row + (size_t)head * hd;
    const float a = to_f32(vec[i0]), bb = to_f32(vec[i1]);
    vec[i0] = from_f32<T>(a * cs[k] - bb * cs[half + k]);
    vec[i1] = from_f32<T>(a * cs[half + k] + bb * cs[k]);
  }
  if (!store || kv0 >= h1) return;
  __syncthreads();                                      // the rotated keys are read back below
  for (int i = threadIdx.x; i < (h1 - kv0) * hd; i += blockDim.x) {
    const int hh = kv0 + i / hd - heads, d = i % hd;    // hh in [0, 2 nkv): keys then values
    const bool is_k = hh < nkv;
    const int kvh = is_k ? hh : hh - nkv;
    const long long off = kv_row_offset(c, slot, pos, kvh, err);
    if (off < 0) continue;
    ((T*)(is_k ? c.k : c.v))[off + d] = row[(size_t)(heads + hh) * hd + d];
  }
}

IERT_API int iert_rope_kv_store(void* qkv, int dtype, const IertBatchView* batch,
                                const IertKvView* cache, const float* inv_freq, int heads,
                                int rotary_dim, int pairing, int write_cache, int* err,
                                cudaStream_t stream) {
  if (batch->n_tokens <= 0) return IERT_OK;
  if (rotary_dim < 0 || rotary_dim > cache->head_dim || (rotary_dim & 1) || cache->dtype != dtype)
    return IERT_BAD_ARGUMENT;
  if (pairing != IERT_PAIR_HALF && pairing != IERT_PAIR_INTERLEAVED) return IERT_BAD_ARGUMENT;
  // few tokens: spread the heads over many blocks; many tokens: one block per token
  const int total_heads = heads + 2 * cache->kv_heads;
  const int heads_per_block = batch->n_tokens >= 512 ? total_heads : (total_heads >= 8 ? 8 : total_heads);
  const int work = heads_per_block * (rotary_dim / 2 > 0 ? rotary_dim / 2 : 1);
  const int threads = work >= 2048 ? 256 : work >= 512 ? 128 : 64;
  const size_t smem = (size_t)rotary_dim * sizeof(float);
  if (smem > 48 * 1024) return IERT_BAD_ARGUMENT;
  dim3 grid(batch->n_tokens, (total_heads + heads_per_block - 1) / heads_per_block);
  // bf16, every head a whole number of 16-byte runs, and the rotated part too
  const int hd = cache->head_dim;
  const int vec8 = dtype == IERT_BF16 && hd % 8 == 0 && rotary_dim % (pairing == IERT_PAIR_HALF ? 16 : 8) == 0 &&
                   (((uintptr_t)qkv | (uintptr_t)cache->k | (uintptr_t)cache->v) & 15) == 0;
  if (dtype == IERT_F32)
    launch_dep(rope_kv_store_kernel<float>, grid, dim3(threads), smem, stream, (float*)qkv, *batch, *cache, inv_freq, heads, rotary_dim, pairing, write_cache, heads_per_block, 0, err);
  else if (dtype == IERT_BF16)
    launch_dep(rope_kv_store_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, (__nv_bfloat16*)qkv, *batch, *cache, inv_freq, heads, rotary_dim, pairing, write_cache, heads_per_block, vec8, err);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("rope_kv_store");
}

// ---------------------------------------------------------------------------------------
// SwiGLU activation on a fused [T, 2*I] projection: out[t, i] = silu(gu[t, i]) * gu[t, I+i],
// sigmoid evaluated on the stable branch.  Reference: src/ops/swiglu.rs:3-36.
__device__ __forceinline__ float stable_sigmoid(float x) {
  if (x >= 0.f) return 1.0f / (1.0f + expf(-x));
  const float z = expf(x);
  return z / (1.0f + z);
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                                size_t total) {
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_f32(gu[t * 2 * inter + i]);
    const float u = to_f32(gu[t * 2 * inter + inter + i]);
    out[idx] = from_f32<T>(g * stable_sigmoid(g) * u);
  }
}

// bf16, 8 elements (16 bytes) per thread; `inter` a multiple of 8.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       int inter, size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = inter / 8;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / per_row;
    const int i = (int)(idx - t * per_row) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + i);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + i);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(gp[e]), u = __bfloat1622float2(up[e]);
      op[e] = __floats2bfloat162_rn(g.x * stable_sigmoid(g.x) * u.x, g.y * stable_sigmoid(g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inter + i) = o4;
  }
}

IERT_API int iert_silu_mul(const void* gu, void* out, int dtype, int n_tokens, int inter,
                           cudaStream_t stream) {
  if (n_tokens <= 0) return IERT_OK;
  if (inter <= 0) return IERT_BAD_ARGUMENT;
  const size_t total = (size_t)n_tokens * inter;
  const int threads = 256;
  if (dtype == IERT_BF16 && inter % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const size_t total8 = total / 8;
    const size_t want = (total8 + threads - 1) / threads;
    const size_t cap = (size_t)iert_sm_count_cached() * 32;
    const int blocks = (int)(want < cap ? want : cap);
    launch_dep(silu_mul_bf16x8_kernel, blocks, threads, 0, stream, (const __nv_bfloat16*)gu,
               (__nv_bfloat16*)out, inter, total8);
    return iert_check_launch("silu_mul");
  }
  const size_t cap16 = (size_t)iert_sm_count_cached() * 16;
  const int blocks = (int)((total + threads - 1) / threads < cap16 ? (total + threads - 1) / threads : cap16);
  if (dtype == IERT_F32)
    launch_dep(silu_mul_kernel<float>, blocks, threads, 0, stream, (const float*)gu, (float*)out, inter, total);
  else if (dtype == IERT_BF16)
    launch_dep(silu_mul_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("silu_mul");
}

// ---------------------------------------------------------------------------------------
// residual[i] += y[i] in fp32 (src/ops/residual_add.rs:3-12).  Used by parts whose last
// kernel cannot add into the residual stream itself.
template <typename T>
__global__ void add_into_kernel(float* __restrict__ residual, const T* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    residual[i] += to_f32(y[i]);
}

IERT_API int iert_add_into(float* residual, const void* y, int y_dtype, long long n,
                           cudaStream_t stream) {
  if (n <= 0) return IERT_OK;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const long long cap = (long long)iert_sm_count_cached() * 16;
  const int blocks = (int)(want < cap ? want : cap);
  if (y_dtype == IERT_F32)
    add_into_kernel<float><<<blocks, threads, 0, stream>>>(residual, (const float*)y, (size_t)n);
  else if (y_dtype == IERT_BF16)
    add_into_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(residual, (const __nv_bfloat16*)y, (size_t)n);
  else
    return IERT_BAD_ARGUMENT;
  return iert_check_launch("add_into");
}

// ---------------------------------------------------------------------------------------
// After a step: pos0[s] += tokens the sequence brought, so that the same device-resident
// batch description can drive the next one-token step without the host.
__global__ void advance_positions_kernel(int* __restrict__ pos0, const int* __restrict__ cu_q,
                                         const int* __restrict__ slot_ids, int n_seqs) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_seqs) return;
  if (slot_ids[s] >= 0) pos0[s] += cu_q[s + 1] - cu_q[s];
}

IERT_API int iert_advance_positions(int* pos0, const int* cu_q, const int* slot_ids, int n_seqs,
                                    cudaStream_t stream) {
  if (n_seqs <= 0) return IERT_OK;
  advance_positions_kernel<<<(n_seqs + 127) / 128, 128, 0, stream>>>(pos0, cu_q, slot_ids, n_seqs);
  return iert_check_launch("advance_positions");
}
