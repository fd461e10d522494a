// Next-token choice on the device: greedy (first largest logit) and temperature sampling
// by inverse CDF in vocabulary order, with one Philox4x32-10 draw per (request, step).
// Reference: src/engine/sampling.rs:25-38 (argmax, first index wins a tie, non-finite
// logits are an error), :54-79 (softmax(logits / T), r in [0,1), first i with r < cum_i,
// else the last index).
#include "common.cuh"

using namespace iert;

namespace {

constexpr int THREADS = 1024;

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// The uniform draw of request `request` at decoding step `step` under `seed`: the first
// output word's top 24 bits, in [0, 1).  It depends on nothing else, so a request samples
// the same alone or in any batch.
__device__ __forceinline__ float uniform_draw(uint64_t seed, uint32_t request, uint32_t step) {
  uint32_t c[4] = {request, step, 0u, 0u};
  philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, long long ld, int* __restrict__ out,
              int* __restrict__ err) {
  __shared__ float vs[32];
  __shared__ int is[32];
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  const float* row = logits + (long long)blockIdx.x * ld;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int i = threadIdx.x; i < vocab; i += THREADS) {
    const float v = row[i];
    if (!isfinite(v)) bad = true;
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  if (bad) atomicOr(err, IERT_ERR_NONFINITE_LOGIT);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { vs[warp] = best; is[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = vs[lane]; best_i = is[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

// Thread t owns the contiguous ids [t*chunk, (t+1)*chunk).  Sums: each thread adds its
// chunk in id order; thread totals are scanned in thread order.  The chosen id is the
// first one whose running sum exceeds r * total.
__global__ void __launch_bounds__(THREADS)
temperature_kernel(const float* __restrict__ logits, int vocab, long long ld, float temperature,
                   uint64_t seed, const int* __restrict__ request_ids,
                   const int* __restrict__ step_ids, int* __restrict__ out,
                   int* __restrict__ err) {
  __shared__ float scratch[33];
  __shared__ float warp_tot[32];
  __shared__ int owner;
  pdl_launch_dependents();     // the next kernel may start its preamble now
  pdl_wait();                  // everything below may depend on the kernel before
  const float* row = logits + (long long)blockIdx.x * ld;
  const int chunk = (vocab + THREADS - 1) / THREADS;
  const int lo = min(vocab, (int)threadIdx.x * chunk), hi = min(vocab, lo + chunk);

  float mx = -INFINITY;
  bool bad = false;
  for (int i = lo; i < hi; ++i) {
    const float v = row[i];
    if (!isfinite(v)) bad = true;
    mx = fmaxf(mx, v / temperature);
  }
  if (bad) atomicOr(err, IERT_ERR_NONFINITE_LOGIT);
  mx = block_max(mx, scratch);

  float local = 0.f;
  for (int i = lo; i < hi; ++i) local += expf(row[i] / temperature - mx);

  // Boundaries: lower[t] = sum of the totals of threads before t (warp scan, then a scan
  // of the warp totals).  The owner of the draw is the LAST thread with a non-empty chunk
  // whose lower boundary is <= target, so rounding in the scans can never leave the
  // target between two chunks.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  float excl = __shfl_up_sync(0xffffffffu, incl, 1);
  if (lane == 0) excl = 0.f;
  if (lane == 31) warp_tot[warp] = incl;
  if (threadIdx.x == 0) owner = -1;
  __syncthreads();
  if (warp == 0) {
    float w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += up;
    }
    warp_tot[lane] = w;                      // inclusive over warps
  }
  __syncthreads();
  const float lower = (warp > 0 ? warp_tot[warp - 1] : 0.f) + excl;
  const float total = warp_tot[31];

  const float r = uniform_draw(seed, (uint32_t)request_ids[blockIdx.x], (uint32_t)step_ids[blockIdx.x]);
  const float target = r * total;
  if (hi > lo && lower <= target) atomicMax(&owner, (int)threadIdx.x);
  __syncthreads();
  if ((int)threadIdx.x == owner) {
    float cum = lower;
    int pick = hi - 1;
    for (int i = lo; i < hi; ++i) {
      cum += expf(row[i] / temperature - mx);
      if (target < cum) { pick = i; break; }
    }
    out[blockIdx.x] = pick;
  }
  if (threadIdx.x == 0 && owner < 0) out[blockIdx.x] = vocab - 1;
}

__global__ void uniform_kernel(uint64_t seed, const int* request_ids, const int* step_ids,
                               float* out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = uniform_draw(seed, (uint32_t)request_ids[i], (uint32_t)step_ids[i]);
}

}  // namespace

// logits: [rows, vocab] fp32 with row stride ld.  out: [rows] int32.
IERT_API int iert_sample_greedy(const float* logits, int rows, int vocab, long long ld, int* out,
                                int* err, cudaStream_t stream) {
  if (rows <= 0) return IERT_OK;
  if (vocab <= 0) return IERT_BAD_ARGUMENT;
  launch_dep(argmax_kernel, rows, THREADS, 0, stream, logits, vocab, ld, out, err);
  return iert_check_launch("sample_greedy");
}

IERT_API int iert_sample_temperature(const float* logits, int rows, int vocab, long long ld,
                                     float temperature, unsigned long long seed,
                                     const int* request_ids, const int* step_ids, int* out,
                                     int* err, cudaStream_t stream) {
  if (rows <= 0) return IERT_OK;
  if (vocab <= 0 || !(temperature > 0.f) || !isfinite(temperature)) return IERT_BAD_ARGUMENT;
  launch_dep(temperature_kernel, rows, THREADS, 0, stream, logits, vocab, ld, temperature, seed,
                                                   request_ids, step_ids, out, err);
  return iert_check_launch("sample_temperature");
}

// The draws themselves, for tests and for callers that want to sample elsewhere.
IERT_API int iert_uniform_draws(unsigned long long seed, const int* request_ids,
                                const int* step_ids, float* out, int n, cudaStream_t stream) {
  if (n <= 0) return IERT_OK;
  uniform_kernel<<<(n + 127) / 128, 128, 0, stream>>>(seed, request_ids, step_ids, out, n);
  return iert_check_launch("uniform_draws");
}
