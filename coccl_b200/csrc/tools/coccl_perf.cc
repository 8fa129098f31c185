// coccl-perf: collective benchmark through the public C API, one process, one thread per GPU.
//
//   coccl-perf -o all_reduce -g 8 -b 1M -e 1G -f 2 -d float -w 5 -n 20 [-c 1] [-x explicit]
//
// What the reference ships as a family of nccl-tests programs (all_reduce_perf, all_reduce_comp_oneshot_perf, ...;
// tests/coccl-tests/src/Makefile:97-101, protocol of examples/benchmarks_scripts/communication_benchmarks.sh) is one
// program here: -o picks the collective, -x the entry point (the standard call, which the policy file routes, or
// one of the explicit compressed calls). COCCL_ENABLE / COCCL_CONFIG_FILE choose the policy; with COCCL_ENABLE=0 the
// same command measures the installed NCCL. Sizes are logical bytes (all-reduce: the buffer; the other operations:
// the total over all ranks), bus bandwidth follows the nccl-tests conventions. With -c 1 the result of the first
// call of every size is compared with a host-computed reference and the relative RMS error is printed.
//
// Timing: a barrier between the threads, then -n calls bracketed by CUDA events on every rank's stream; the reported
// time is the slowest rank's average. With -F 1 every call is timed on its own after a 256 MiB write (cold L2).
#include <cuda_runtime.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "coccl/coccl.h"

namespace {

enum class Op { AllReduce, ReduceScatter, AllGather, AllToAll };
enum class Entry { Standard, OneShot, TwoShot, TripleShot, Explicit };

struct Options {
  Op op = Op::AllReduce;
  Entry entry = Entry::Standard;
  int gpus = 0, warmup = 5, iters = 20, check = 0, flush = 0;
  size_t minBytes = 1u << 20, maxBytes = 64u << 20;
  double factor = 2.0;
  ncclDataType_t dtype = ncclFloat32;
  std::string opName = "all_reduce", dtypeName = "float", entryName = "standard";
};

bool parseSize(const char* text, size_t* out) {
  char* end = nullptr;
  const double v = strtod(text, &end);
  if (end == text || v < 0) return false;
  double scale = 1;
  switch (*end) {
    case 0: break;
    case 'k': case 'K': scale = 1024.0; break;
    case 'm': case 'M': scale = 1024.0 * 1024; break;
    case 'g': case 'G': scale = 1024.0 * 1024 * 1024; break;
    default: return false;
  }
  *out = (size_t)(v * scale);
  return true;
}

int usage(const char* why) {
  if (why) fprintf(stderr, "coccl-perf: %s\n", why);
  fprintf(stderr,
          "usage: coccl-perf [-o all_reduce|reduce_scatter|all_gather|alltoall] [-x standard|oneshot|twoshot|tripleshot|explicit]\n"
          "                  [-g gpus] [-b min] [-e max] [-f factor] [-d float|half|bfloat16] [-w warmup] [-n iterations] [-c 0|1] [-F 0|1]\n"
          "  sizes take K, M, G suffixes; -x oneshot/twoshot/tripleshot select cocclAllReduceComp* / cocclReduceScatterComp*,\n"
          "  -x explicit selects cocclAllGatherComp / cocclAllToAllComp; policy from COCCL_ENABLE / COCCL_CONFIG_FILE\n"
          "  -F 1 writes a 256 MiB buffer before every timed call (cold L2) and times each call on its own\n");
  return 2;
}

bool parse(int argc, char** argv, Options* o, const char** error) {
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "-h" || a == "--help") { *error = nullptr; return false; }
    if (i + 1 >= argc) { *error = "option without a value"; return false; }
    const char* v = argv[++i];
    if (a == "-o") {
      o->opName = v;
      if (o->opName == "all_reduce") o->op = Op::AllReduce;
      else if (o->opName == "reduce_scatter") o->op = Op::ReduceScatter;
      else if (o->opName == "all_gather") o->op = Op::AllGather;
      else if (o->opName == "alltoall" || o->opName == "all_to_all") o->op = Op::AllToAll;
      else { *error = "unknown operation"; return false; }
    } else if (a == "-x") {
      o->entryName = v;
      if (o->entryName == "standard") o->entry = Entry::Standard;
      else if (o->entryName == "oneshot") o->entry = Entry::OneShot;
      else if (o->entryName == "twoshot") o->entry = Entry::TwoShot;
      else if (o->entryName == "tripleshot") o->entry = Entry::TripleShot;
      else if (o->entryName == "explicit") o->entry = Entry::Explicit;
      else { *error = "unknown entry point"; return false; }
    } else if (a == "-g") o->gpus = atoi(v);
    else if (a == "-w") o->warmup = atoi(v);
    else if (a == "-n") o->iters = atoi(v);
    else if (a == "-c") o->check = atoi(v);
    else if (a == "-F") o->flush = atoi(v);
    else if (a == "-f") o->factor = atof(v);
    else if (a == "-b") { if (!parseSize(v, &o->minBytes)) { *error = "bad -b"; return false; } }
    else if (a == "-e") { if (!parseSize(v, &o->maxBytes)) { *error = "bad -e"; return false; } }
    else if (a == "-d") {
      o->dtypeName = v;
      if (o->dtypeName == "float") o->dtype = ncclFloat32;
      else if (o->dtypeName == "half") o->dtype = ncclFloat16;
      else if (o->dtypeName == "bfloat16") o->dtype = ncclBfloat16;
      else { *error = "unknown datatype"; return false; }
    } else { *error = "unknown option"; return false; }
  }
  if (o->iters < 1 || o->warmup < 0 || o->factor <= 1.0 || o->minBytes == 0 || o->maxBytes < o->minBytes) { *error = "bad range or counts"; return false; }
  const bool reduction = o->op == Op::AllReduce || o->op == Op::ReduceScatter;
  if ((o->entry == Entry::OneShot || o->entry == Entry::TwoShot) && !reduction) { *error = "-x oneshot/twoshot need a reduction"; return false; }
  if (o->entry == Entry::TripleShot && o->op != Op::AllReduce) { *error = "-x tripleshot needs all_reduce"; return false; }
  if (o->entry == Entry::Explicit && reduction) { *error = "-x explicit is for all_gather / alltoall"; return false; }
  return true;
}

size_t widthOf(ncclDataType_t t) { return t == ncclFloat32 ? 4 : 2; }

// Values of rank r at index i: small, different per rank, exactly representable in every datatype offered.
float valueAt(int rank, size_t i) { return (float)((int)((i * 7 + (size_t)rank * 13) % 61) - 30) / 64.0f; }

uint16_t toHalf(float f) {   // the values above need no rounding: |f| < 1, multiples of 1/64
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int exp = (int)((x >> 23) & 0xff) - 127 + 15;
  const uint32_t man = (x >> 13) & 0x3ffu;
  if ((x & 0x7fffffffu) == 0) return (uint16_t)sign;
  if (exp <= 0) return (uint16_t)(sign | ((man | 0x400u) >> (1 - exp)));
  return (uint16_t)(sign | ((uint32_t)exp << 10) | man);
}
uint16_t toBf16(float f) { uint32_t x; memcpy(&x, &f, 4); return (uint16_t)(x >> 16); }
float fromHalf(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  int exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) { x = sign; }
    else {
      exp = 1;
      while ((man & 0x400u) == 0) { man <<= 1; --exp; }
      x = sign | ((uint32_t)(exp + 127 - 15) << 23) | ((man & 0x3ffu) << 13);
    }
  } else {
    x = sign | ((uint32_t)(exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &x, 4);
  return f;
}
float fromBf16(uint16_t b) { uint32_t x = (uint32_t)b << 16; float f; memcpy(&f, &x, 4); return f; }

void encodeHost(ncclDataType_t t, const std::vector<float>& src, std::vector<uint8_t>* dst) {
  dst->resize(src.size() * widthOf(t));
  if (t == ncclFloat32) { memcpy(dst->data(), src.data(), dst->size()); return; }
  uint16_t* p = reinterpret_cast<uint16_t*>(dst->data());
  for (size_t i = 0; i < src.size(); ++i) p[i] = t == ncclFloat16 ? toHalf(src[i]) : toBf16(src[i]);
}
void decodeHost(ncclDataType_t t, const std::vector<uint8_t>& src, std::vector<float>* dst) {
  dst->resize(src.size() / widthOf(t));
  if (t == ncclFloat32) { memcpy(dst->data(), src.data(), src.size()); return; }
  const uint16_t* p = reinterpret_cast<const uint16_t*>(src.data());
  for (size_t i = 0; i < dst->size(); ++i) (*dst)[i] = t == ncclFloat16 ? fromHalf(p[i]) : fromBf16(p[i]);
}

struct Shared {
  Options opt;
  int n = 0;
  std::vector<ncclComm_t> comms;
  pthread_barrier_t barrier;
  std::vector<double> ms;       // per rank, per size: average time of a call
  std::vector<double> err2, ref2;
  std::vector<int> failed;
};

struct Job { Shared* s; int rank; };

// send / receive element counts per rank and the count argument of the call, for `bytes` logical bytes
void shapeOf(const Options& o, int n, size_t bytes, size_t* sendCount, size_t* recvCount, size_t* arg) {
  const size_t w = widthOf(o.dtype);
  size_t total = bytes / w;
  total -= total % ((size_t)n * n ? (size_t)n * n : 1);   // divisible for every operation
  if (total == 0) total = (size_t)n * n;
  switch (o.op) {
    case Op::AllReduce: *sendCount = *recvCount = *arg = total; break;
    case Op::ReduceScatter: *sendCount = total; *recvCount = *arg = total / n; break;
    case Op::AllGather: *sendCount = *arg = total / n; *recvCount = total; break;
    case Op::AllToAll: *sendCount = *recvCount = total / n; *arg = total / n / n; break;
  }
}

ncclResult_t issue(const Options& o, const void* send, void* recv, size_t arg, ncclComm_t comm, cudaStream_t st) {
  switch (o.op) {
    case Op::AllReduce:
      if (o.entry == Entry::OneShot) return cocclAllReduceCompOneShot(send, recv, arg, o.dtype, ncclSum, comm, st);
      if (o.entry == Entry::TwoShot) return cocclAllReduceCompTwoShot(send, recv, arg, o.dtype, ncclSum, comm, st);
      if (o.entry == Entry::TripleShot) return cocclAllReduceCompTripleShot(send, recv, arg, o.dtype, ncclSum, comm, st);
      return cocclApiAllReduce(send, recv, arg, o.dtype, ncclSum, comm, st);
    case Op::ReduceScatter:
      if (o.entry == Entry::OneShot) return cocclReduceScatterCompOneShot(send, recv, arg, o.dtype, ncclSum, comm, st);
      if (o.entry == Entry::TwoShot) return cocclReduceScatterCompTwoShot(send, recv, arg, o.dtype, ncclSum, comm, st);
      return cocclApiReduceScatter(send, recv, arg, o.dtype, ncclSum, comm, st);
    case Op::AllGather:
      if (o.entry == Entry::Explicit) return cocclAllGatherComp(send, recv, arg, o.dtype, comm, st);
      return cocclApiAllGather(send, recv, arg, o.dtype, comm, st);
    case Op::AllToAll:
      if (o.entry == Entry::Explicit) return cocclAllToAllComp(send, recv, arg, o.dtype, comm, st);
      return cocclApiAllToAll(send, recv, arg, o.dtype, comm, st);
  }
  return ncclInvalidArgument;
}

// what rank `rank` must hold at receive index i
float expected(const Options& o, int n, int rank, size_t i, size_t sendCount, size_t recvCount) {
  switch (o.op) {
    case Op::AllReduce: { float s = 0; for (int r = 0; r < n; ++r) s += valueAt(r, i); return s; }
    case Op::ReduceScatter: { float s = 0; for (int r = 0; r < n; ++r) s += valueAt(r, (size_t)rank * recvCount + i); return s; }
    case Op::AllGather: return valueAt((int)(i / sendCount), i % sendCount);
    case Op::AllToAll: { const size_t per = sendCount / n; return valueAt((int)(i / per), (size_t)rank * per + i % per); }
  }
  return 0;
}

std::vector<size_t> sizesOf(const Options& o) {
  std::vector<size_t> v;
  for (double b = (double)o.minBytes; b <= (double)o.maxBytes * 1.0000001; b *= o.factor) v.push_back((size_t)b);
  return v;
}

void* worker(void* arg) {
  Job* job = static_cast<Job*>(arg);
  Shared& s = *job->s;
  const Options& o = s.opt;
  const int rank = job->rank, n = s.n;
  auto fail = [&](const char* what, int code) {
    fprintf(stderr, "coccl-perf: rank %d: %s failed (%d)\n", rank, what, code);
    s.failed[rank] = 1;
  };
  if (cudaSetDevice(rank) != cudaSuccess) { fail("cudaSetDevice", 0); }
  cudaStream_t stream = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  const std::vector<size_t> sizes = sizesOf(o);
  size_t maxSend = 0, maxRecv = 0;
  for (size_t b : sizes) {
    size_t sc, rc, a;
    shapeOf(o, n, b, &sc, &rc, &a);
    if (sc > maxSend) maxSend = sc;
    if (rc > maxRecv) maxRecv = rc;
  }
  void *send = nullptr, *recv = nullptr, *flushBuffer = nullptr;
  const size_t kFlushBytes = 256u << 20;
  if (o.flush && cudaMalloc(&flushBuffer, kFlushBytes) != cudaSuccess) fail("cudaMalloc", 0);
  const size_t w = widthOf(o.dtype);
  if (cudaMalloc(&send, maxSend * w) != cudaSuccess || cudaMalloc(&recv, maxRecv * w) != cudaSuccess) fail("cudaMalloc", 0);
  std::vector<float> host;
  std::vector<uint8_t> raw;
  for (size_t k = 0; k < sizes.size(); ++k) {
    size_t sc, rc, a;
    shapeOf(o, n, sizes[k], &sc, &rc, &a);
    if (!s.failed[rank]) {
      host.resize(sc);
      for (size_t i = 0; i < sc; ++i) host[i] = valueAt(rank, i);
      encodeHost(o.dtype, host, &raw);
      if (cudaMemcpy(send, raw.data(), raw.size(), cudaMemcpyHostToDevice) != cudaSuccess) fail("cudaMemcpy", 0);
    }
    pthread_barrier_wait(&s.barrier);
    bool anyFailed = false;
    for (int r = 0; r < n; ++r) anyFailed = anyFailed || s.failed[r];
    if (anyFailed) break;   // every thread sees the same flags after the barrier: all leave together
    ncclResult_t rcode = ncclSuccess;
    for (int i = 0; i < o.warmup + 1 && rcode == ncclSuccess; ++i) {
      rcode = issue(o, send, recv, a, s.comms[rank], stream);
      if (i == 0 && rcode == ncclSuccess && o.check) {
        cudaStreamSynchronize(stream);
        raw.resize(rc * w);
        cudaMemcpy(raw.data(), recv, raw.size(), cudaMemcpyDeviceToHost);
        decodeHost(o.dtype, raw, &host);
        double e2 = 0, r2 = 0;
        const size_t stride = rc > (1u << 20) ? rc / (1u << 20) : 1;   // at most about a million samples
        for (size_t i2 = 0; i2 < rc; i2 += stride) {
          const double want = expected(o, n, rank, i2, sc, rc);
          e2 += (host[i2] - want) * (host[i2] - want);
          r2 += want * want;
        }
        s.err2[rank * sizes.size() + k] = e2;
        s.ref2[rank * sizes.size() + k] = r2;
      }
    }
    cudaStreamSynchronize(stream);
    pthread_barrier_wait(&s.barrier);
    float ms = 0;
    if (o.flush && flushBuffer != nullptr) {
      // cold L2: a buffer twice the size of the L2 is overwritten before every call, the ranks meet, and the call
      // is timed on its own; every thread runs all iterations (also after a failure) so that the barriers match
      for (int i = 0; i < o.iters; ++i) {
        cudaMemsetAsync(flushBuffer, i & 0xff, kFlushBytes, stream);
        cudaStreamSynchronize(stream);
        pthread_barrier_wait(&s.barrier);
        cudaEventRecord(e0, stream);
        if (rcode == ncclSuccess) rcode = issue(o, send, recv, a, s.comms[rank], stream);
        cudaEventRecord(e1, stream);
        if (cudaEventSynchronize(e1) != cudaSuccess) fail("cudaEventSynchronize", 0);
        float one = 0;
        cudaEventElapsedTime(&one, e0, e1);
        ms += one;
      }
    } else {
      cudaEventRecord(e0, stream);
      for (int i = 0; i < o.iters && rcode == ncclSuccess; ++i) rcode = issue(o, send, recv, a, s.comms[rank], stream);
      cudaEventRecord(e1, stream);
      if (cudaEventSynchronize(e1) != cudaSuccess) fail("cudaEventSynchronize", 0);
      cudaEventElapsedTime(&ms, e0, e1);
    }
    s.ms[rank * sizes.size() + k] = ms / o.iters;
    if (rcode != ncclSuccess) fail(cocclApiGetErrorString(rcode), (int)rcode);
    ncclResult_t async = ncclSuccess;
    if (cocclApiCommGetAsyncError(s.comms[rank], &async) == ncclSuccess && async != ncclSuccess) fail("asynchronous error", (int)async);
  }
  if (send) cudaFree(send);
  if (recv) cudaFree(recv);
  if (flushBuffer) cudaFree(flushBuffer);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamDestroy(stream);
  return nullptr;
}

}  // namespace

int main(int argc, char** argv) {
  Shared s;
  const char* error = nullptr;
  if (!parse(argc, argv, &s.opt, &error)) return usage(error);
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices < 1) {
    fprintf(stderr, "coccl-perf: no CUDA device\n");
    return 1;
  }
  s.n = s.opt.gpus > 0 ? s.opt.gpus : devices;
  if (s.n < 2 || s.n > devices) { fprintf(stderr, "coccl-perf: %d GPUs asked for, %d present (at least 2 are needed)\n", s.n, devices); return 1; }
  s.comms.resize(s.n);
  ncclResult_t r = cocclApiCommInitAll(s.comms.data(), s.n, nullptr);
  if (r != ncclSuccess) { fprintf(stderr, "coccl-perf: ncclCommInitAll: %s\n", cocclApiGetErrorString(r)); return 1; }
  const std::vector<size_t> sizes = sizesOf(s.opt);
  s.ms.assign(sizes.size() * s.n, 0.0);
  s.err2.assign(sizes.size() * s.n, 0.0);
  s.ref2.assign(sizes.size() * s.n, 0.0);
  s.failed.assign(s.n, 0);
  pthread_barrier_init(&s.barrier, nullptr, s.n);
  std::vector<pthread_t> threads(s.n);
  std::vector<Job> jobs(s.n);
  for (int i = 0; i < s.n; ++i) { jobs[i] = Job{&s, i}; pthread_create(&threads[i], nullptr, worker, &jobs[i]); }
  for (int i = 0; i < s.n; ++i) pthread_join(threads[i], nullptr);
  int bad = 0;
  for (int f : s.failed) bad += f;
  const char* enabled = getenv("COCCL_ENABLE");
  printf("# coccl-perf op=%s entry=%s dtype=%s gpus=%d warmup=%d iterations=%d COCCL_ENABLE=%s COCCL_CONFIG_FILE=%s\n",
         s.opt.opName.c_str(), s.opt.entryName.c_str(), s.opt.dtypeName.c_str(), s.n, s.opt.warmup, s.opt.iters,
         enabled ? enabled : "(unset)", getenv("COCCL_CONFIG_FILE") ? getenv("COCCL_CONFIG_FILE") : "(unset)");
  printf("# %12s %12s %10s %10s %10s %12s\n", "bytes", "elements", "time_us", "algbw_GBs", "busbw_GBs", "rel_rms_err");
  for (size_t k = 0; k < sizes.size() && !bad; ++k) {
    size_t sc, rc, a;
    shapeOf(s.opt, s.n, sizes[k], &sc, &rc, &a);
    const size_t total = s.opt.op == Op::AllReduce ? sc : (s.opt.op == Op::AllToAll ? sc * s.n : (sc > rc ? sc : rc));
    double ms = 0, e2 = 0, r2 = 0;
    for (int rk = 0; rk < s.n; ++rk) {
      if (s.ms[rk * sizes.size() + k] > ms) ms = s.ms[rk * sizes.size() + k];
      e2 += s.err2[rk * sizes.size() + k];
      r2 += s.ref2[rk * sizes.size() + k];
    }
    const double bytes = (double)total * widthOf(s.opt.dtype);
    const double alg = bytes / (ms * 1e-3) / 1e9;
    const double bus = alg * (s.opt.op == Op::AllReduce ? 2.0 * (s.n - 1) / s.n : (double)(s.n - 1) / s.n);
    if (s.opt.check) printf("  %12.0f %12zu %10.1f %10.2f %10.2f %12.3e\n", bytes, total, ms * 1e3, alg, bus, r2 > 0 ? sqrt(e2 / r2) : 0.0);
    else printf("  %12.0f %12zu %10.1f %10.2f %10.2f %12s\n", bytes, total, ms * 1e3, alg, bus, "-");
  }
  cocclApiStats st;
  cocclApiGetStats(&st);
  printf("# calls: compressed %llu (fused kernels %llu, staged pipeline %llu), native %llu\n", st.compressedCalls, st.fusedCalls,
         st.stagedCalls, st.nativeCalls);
  if (st.stagedCalls) {
    unsigned long long a = 0, b = 0, c = 0;
    cocclApiStagedReasons(&a, &b, &c);
    printf("# staged because: no fused form %llu, set-up failed %llu, after a failed set-up %llu\n", a, c, b);
  }
  for (int i = 0; i < s.n; ++i) cocclApiCommDestroy(s.comms[i]);
  pthread_barrier_destroy(&s.barrier);
  if (bad) { fprintf(stderr, "coccl-perf: %d rank(s) failed\n", bad); return 1; }
  return 0;
}
