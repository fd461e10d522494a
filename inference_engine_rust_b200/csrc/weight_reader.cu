// Reads byte ranges of a file straight into device memory (or, for tests without a device, into
// host memory): the tensor data of a safetensors file, each tensor to the place where the model
// keeps it.
//
// The reference opens a weights file once, sorts the wanted tensors by their offset and reads them
// in that order (src/model_loader/gguf_types.rs:200-241).  Here the wanted ranges are cut into
// chunks, in file order, and a few host threads take chunks in turn: each reads its chunk with
// pread into one of its two page-locked buffers and sends it on with an asynchronous copy on a
// stream of its own, so that reading the next chunk overlaps the copy of the one before, and the
// threads together use the host's memory bandwidth and the link to the device, which one thread
// copying out of a mapping cannot.  No tensor passes through the Python heap.
//
// Host code only; no kernel is launched.
#include "common.cuh"

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

struct Chunk {
  long long file_off;
  long long bytes;
  char* dst;
};

struct Job {
  int fd = -1;
  int device = -1;                 // < 0: destinations are host memory, no CUDA call is made
  long long chunk_bytes = 0;
  std::vector<Chunk> chunks;
  std::atomic<size_t> next{0};
  std::atomic<bool> failed{false};
  std::mutex mu;
  std::string error;
  int code = 0;                    // 2: the file, 3: a CUDA call

  void fail(int why, const std::string& msg) {
    std::lock_guard<std::mutex> g(mu);
    if (!failed.exchange(true)) { code = why; error = msg; }
  }
};

// Reads exactly `n` bytes at `off`; false with `why` set when the file ends early or a read fails.
bool read_fully(int fd, char* buf, long long n, long long off, std::string* why) {
  long long got = 0;
  while (got < n) {
    ssize_t r = pread(fd, buf + got, (size_t)(n - got), (off_t)(off + got));
    if (r < 0) {
      if (errno == EINTR) continue;
      *why = std::string("read failed at byte ") + std::to_string(off + got) + ": " + strerror(errno);
      return false;
    }
    if (r == 0) {
      *why = "the file ends at byte " + std::to_string(off + got) + ", inside a tensor's data";
      return false;
    }
    got += r;
  }
  return true;
}

void host_worker(Job* job) {
  std::string why;
  for (;;) {
    const size_t i = job->next.fetch_add(1);
    if (i >= job->chunks.size() || job->failed.load()) return;
    const Chunk& c = job->chunks[i];
    if (!read_fully(job->fd, c.dst, c.bytes, c.file_off, &why)) { job->fail(2, why); return; }
  }
}

void device_worker(Job* job) {
  auto cuda_fail = [&](const char* what, cudaError_t e) {
    job->fail(3, std::string(what) + ": " + cudaGetErrorString(e));
  };
  cudaError_t e = cudaSetDevice(job->device);
  if (e != cudaSuccess) { cuda_fail("cudaSetDevice", e); return; }
  char* buf[2] = {nullptr, nullptr};
  cudaEvent_t ev[2] = {nullptr, nullptr};
  bool used[2] = {false, false};
  cudaStream_t stream = nullptr;
  e = cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) { cuda_fail("cudaStreamCreate", e); return; }
  for (int b = 0; b < 2 && e == cudaSuccess; ++b) {
    e = cudaHostAlloc((void**)&buf[b], (size_t)job->chunk_bytes, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ev[b], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) cuda_fail("page-locked staging buffers", e);
  std::string why;
  int turn = 0;
  while (e == cudaSuccess) {
    const size_t i = job->next.fetch_add(1);
    if (i >= job->chunks.size() || job->failed.load()) break;
    const Chunk& c = job->chunks[i];
    const int b = turn++ & 1;
    if (used[b]) {                                   // the copy that last used this buffer must be over
      e = cudaEventSynchronize(ev[b]);
      if (e != cudaSuccess) { cuda_fail("waiting for a copy", e); break; }
    }
    if (!read_fully(job->fd, buf[b], c.bytes, c.file_off, &why)) { job->fail(2, why); break; }
    e = cudaMemcpyAsync(c.dst, buf[b], (size_t)c.bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(ev[b], stream);
    if (e != cudaSuccess) { cuda_fail("copy to the device", e); break; }
    used[b] = true;
  }
  cudaError_t s = cudaStreamSynchronize(stream);     // also on failure: the buffers are freed below
  if (s != cudaSuccess && !job->failed.load()) cuda_fail("copy to the device", s);
  for (int b = 0; b < 2; ++b) {
    if (ev[b]) cudaEventDestroy(ev[b]);
    if (buf[b]) cudaFreeHost(buf[b]);
  }
  cudaStreamDestroy(stream);
}

void put_error(char* err, int err_len, const std::string& msg) {
  if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", msg.c_str());
}

}  // namespace

// Reads `n` ranges of the file at `path`: range i is `bytes[i]` bytes from `file_off[i]`, and
// goes to `dst[i]` (device memory of `device`; host memory when `device` < 0).  `threads` host
// threads (0: as many as the host has, at most 8) take chunks of `chunk_bytes` (0: 4 MiB) in file
// order.  Returns when every byte has arrived.  0 on success; else 1 (bad arguments), 2 (the file
// cannot be opened or read, or ends early) or 3 (a CUDA call failed), with a message in `err`.
IERT_API int iert_read_file_ranges(const char* path, int n, const long long* file_off, const long long* bytes,
                                   void* const* dst, int device, int threads, long long chunk_bytes,
                                   char* err, int err_len) {
  if (!path || n < 0 || (n > 0 && (!file_off || !bytes || !dst)) || threads < 0 || chunk_bytes < 0) {
    put_error(err, err_len, "bad arguments");
    return 1;
  }
  Job job;
  job.device = device;
  job.chunk_bytes = chunk_bytes > 0 ? chunk_bytes : (4ll << 20);     // measured best of 2 to 32 MiB with 8 threads
  // ranges in file order
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](int a, int b) { return file_off[a] < file_off[b]; });
  for (int k = 0; k < n; ++k) {
    const int i = order[k];
    if (file_off[i] < 0 || bytes[i] < 0 || (bytes[i] > 0 && !dst[i])) {
      put_error(err, err_len, "range " + std::to_string(i) + ": negative offset or size, or no destination");
      return 1;
    }
    for (long long done = 0; done < bytes[i]; done += job.chunk_bytes) {
      const long long len = bytes[i] - done < job.chunk_bytes ? bytes[i] - done : job.chunk_bytes;
      job.chunks.push_back({file_off[i] + done, len, (char*)dst[i] + done});
    }
  }
  if (job.chunks.empty()) return 0;
  job.fd = open(path, O_RDONLY | O_CLOEXEC);
  if (job.fd < 0) {
    put_error(err, err_len, std::string("cannot open: ") + strerror(errno));
    return 2;
  }
  if (threads == 0) {
    const unsigned hw = std::thread::hardware_concurrency();
    threads = hw == 0 ? 4 : (hw > 8 ? 8 : (int)hw);
  }
  if ((size_t)threads > job.chunks.size()) threads = (int)job.chunks.size();
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) pool.emplace_back(device < 0 ? host_worker : device_worker, &job);
  for (auto& t : pool) t.join();
  close(job.fd);
  if (!job.failed.load()) return 0;
  put_error(err, err_len, job.error);
  return job.code;
}
