// Shared declarations of the CUDA sources: element types, the cache view that kernels
// receive, status codes and small device helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IERT_API extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
enum : int { IERT_F32 = 0, IERT_BF16 = 1 };

// Status codes returned by every launcher (0 = launched).
enum : int {
  IERT_OK = 0,
  IERT_BAD_ARGUMENT = 1,     // a size or option the kernel does not take
  IERT_CUDA_ERROR = 2,       // the launch itself failed; see iert_last_cuda_error()
};

// Bits that kernels set in the device error word they are given.
enum : int {
  IERT_ERR_TOKEN_RANGE = 1,     // a token id outside [0, vocab)
  IERT_ERR_NONFINITE_LOGIT = 2, // sampling saw NaN or Inf
  IERT_ERR_PAGE_RANGE = 4,      // a page-table entry outside the pool
  IERT_ERR_WAIT_EXPIRED = 8,    // a bounded wait inside a kernel ran out
};

// Rotary pairings: partner of element k.
enum : int { IERT_PAIR_HALF = 0, IERT_PAIR_INTERLEAVED = 1 };

// One layer's keys and values in a paged cache group, plus the page tables of the group.
//   k, v        : [n_pages][kv_heads][page_tokens][head_dim] of `dtype`
//   page_table  : [n_slots][table_width]; logical block b of a sequence is entry
//                 (b % ring_pages) of its row (ring_pages >= table_width means "no ring")
//   window      : 0 = every earlier key is visible; W > 0 = the last W keys, the current
//                 one included
struct IertKvView {
  void* k;
  void* v;
  const int* page_table;
  int table_width;
  int ring_pages;
  int page_tokens;
  int n_pages;
  int kv_heads;
  int head_dim;
  int dtype;
  int window;
};

// The sequences of one step.  All arrays live on the device.
//   cu_q[n_seqs+1] : prefix sums of the tokens each sequence brings
//   slot_ids[n]    : cache slot of each sequence, -1 for a padding sequence
//   tok_seq[T]     : sequence index of each packed token, -1 for a padding token
//   pos0[n]        : tokens each sequence already holds in the cache, before this step
//                    (= the position of the first token it brings)
struct IertBatchView {
  const int* cu_q;
  const int* slot_ids;
  const int* tok_seq;
  const int* pos0;
  int n_seqs;
  int n_tokens;
};

// An RMSNorm split in two around a kernel boundary (one-token steps, where a norm kernel of its own
// costs more than its work).  The kernel that writes new residual rows x[t, :] also writes
//   scaled[t, n] = bf16(x[t, n] * weight[n])          (no row statistic needed: element by element)
//   sumsq[t, p]  = sum of x[t, n]^2 over part p of the row's columns
// (`IertNormAhead`), and the projection that reads `scaled` as its input multiplies its outputs by
// 1 / sqrt(sum_p sumsq[t, p] / hidden + eps) (`IertRowScale`): the product is linear in its input,
// so this is the projection of the normalised row, with one bf16 rounding before the factor instead
// of after it.  Statistics are fp32 and summed in a fixed order.
struct IertNormAhead {
  const void* weight;      // the norm's scale vector [N]
  int weight_dtype;
  void* scaled_out;        // bf16 [M, N], row stride ld
  long long ld;
  float* sumsq_out;        // fp32 [M, parts]; parts is set by the launcher
  int parts;
};
struct IertRowScale {
  const float* sumsq;      // fp32 [M, parts]
  int parts;
  int hidden;              // the length of the normalised rows
  float eps;
};

namespace iert {

// 1 / sqrt(mean + eps) of up to `n_tokens` rows from their partial sums of squares into out[t]
// (shared memory), by a group of `nthreads` threads (a multiple of 32) numbered `tid`: a warp takes
// rows w, w + nwarps, ..., two at a time; a lane loads every 32nd partial sum of both rows, eight
// each before the first is used (one round trip to the L2 for up to 256 parts), adds its own in
// order and the warp adds the lanes by shuffles.  The order of the additions depends on the number
// of parts alone.
__device__ __forceinline__ void row_scales_from_parts(const IertRowScale& rs, int n_tokens, float* out, int tid, int nthreads) {
  const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
  for (int t0 = warp; t0 < n_tokens; t0 += 2 * nwarps) {
    const int t1 = t0 + nwarps;
    const float* p0 = rs.sumsq + (size_t)t0 * rs.parts;
    const float* p1 = rs.sumsq + (size_t)(t1 < n_tokens ? t1 : t0) * rs.parts;
    float s0 = 0.f, s1 = 0.f;
    for (int i0 = lane; i0 < rs.parts; i0 += 256) {
      float a[8], b[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + 32 * j;
        a[j] = i < rs.parts ? __ldcg(p0 + i) : 0.f;
        b[j] = i < rs.parts ? __ldcg(p1 + i) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s0 += a[j]; s1 += b[j]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s0 += __shfl_xor_sync(0xffffffffu, s0, o);
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    }
    if (lane == 0) {
      out[t0] = 1.0f / sqrtf(s0 / (float)rs.hidden + rs.eps);
      if (t1 < n_tokens) out[t1] = 1.0f / sqrtf(s1 / (float)rs.hidden + rs.eps);
    }
  }
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum / max for blocks of up to 1024 threads (blockDim.x a multiple of 32).
// `scratch` holds at least 33 floats.  Every thread gets the result.  The order of the
// additions depends only on blockDim.x, never on the data.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();                 // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Where position `pos` of the sequence in `slot` lives: element offset of its row of
// kv head `h` inside one layer's k or v array.  Returns -1 (and sets the error bit) when
// the page table holds an id outside the pool.
__device__ __forceinline__ long long kv_row_offset(const IertKvView& c, int slot, int pos, int h,
                                                   int* err) {
  const int blk = pos / c.page_tokens;
  const int row = pos - blk * c.page_tokens;
  const int entry = blk % c.ring_pages;
  const int page = c.page_table[(long long)slot * c.table_width + entry];
  if (page < 0 || page >= c.n_pages) {
    if (err) atomicOr(err, IERT_ERR_PAGE_RANGE);
    return -1;
  }
  return (((long long)page * c.kv_heads + h) * c.page_tokens + row) * c.head_dim;
}

// The sequence token t belongs to (-1: padding).  A step with as many tokens as sequences is a
// one-token step: every sequence brings exactly one token and token t is sequence t's, so the
// look-up (one more dependent load at the head of a kernel) is skipped.
__device__ __forceinline__ int sequence_of_token(const IertBatchView& b, int t) {
  return b.n_tokens == b.n_seqs ? t : b.tok_seq[t];
}

// Programmatic dependent launch: a kernel launched with `launch_dep` may start while the
// kernel before it in the stream is still running.  It must call pdl_wait() before it reads
// anything an earlier kernel wrote and before it writes anything an earlier kernel may
// still read; what it does before that (set-up, loads of weights) overlaps the earlier
// kernel.  pdl_launch_dependents() lets the NEXT kernel start its own preamble early.
// Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace iert

// Defined in runtime.cu.
int iert_check_launch(const char* what);
int iert_sm_count_cached();
extern int iert_pdl_enabled;

// Launch `kernel` with programmatic stream serialization (see pdl_wait) when enabled.
template <typename... KArgs, typename... Args>
inline void launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = iert_pdl_enabled ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
