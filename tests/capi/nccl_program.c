/* A plain C program written against the NCCL API only, linked against libcoccl_nccl.so and nothing else of this
 * library: what an application that is relinked (or preloaded) against the drop-in library looks like. The reference
 * reaches PyTorch the same way (examples/training_scripts/train_qwen_coccl.sh:78-82).
 *
 *   nccl_program            version and error strings only (no GPU needed)
 *   nccl_program run N      ncclCommInitAll over N GPUs, in-place all-reduce of 1 Ki and 8 Mi floats, ncclBcast,
 *                           ncclMemAlloc / ncclCommRegister round trip, ncclCommDestroy
 */
#include <cuda_runtime.h>
#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
typedef int ncclDataType_t;
typedef int ncclRedOp_t;
enum { ncclSuccess = 0, ncclFloat32 = 7, ncclSum = 0 };

ncclResult_t ncclGetVersion(int* version);
const char* ncclGetErrorString(ncclResult_t r);
ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist);
ncclResult_t ncclCommCount(ncclComm_t comm, int* n);
ncclResult_t ncclCommUserRank(ncclComm_t comm, int* r);
ncclResult_t ncclCommDestroy(ncclComm_t comm);
ncclResult_t ncclGroupStart(void);
ncclResult_t ncclGroupEnd(void);
ncclResult_t ncclAllReduce(const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st);
ncclResult_t ncclBcast(void* b, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st);
ncclResult_t ncclMemAlloc(void** p, size_t n);
ncclResult_t ncclMemFree(void* p);
ncclResult_t ncclCommRegister(ncclComm_t c, void* b, size_t n, void** h);
ncclResult_t ncclCommDeregister(ncclComm_t c, void* h);
ncclResult_t ncclCommGetAsyncError(ncclComm_t c, ncclResult_t* e);

#define CHECK(x) do { ncclResult_t r_ = (x); if (r_ != ncclSuccess) { printf("FAIL %s -> %d (%s)\n", #x, r_, ncclGetErrorString(r_)); return 1; } } while (0)
#define CU(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("FAIL %s -> %s\n", #x, cudaGetErrorString(e_)); return 1; } } while (0)

/* One thread per GPU issues the collectives (the layout of the reference's benchmarks, `-t N -g 1`,
 * examples/benchmarks_scripts/communication_benchmarks.sh:73): a compressed call may block on its peers during set-up,
 * so the ranks of one process must not be driven from a single thread. */
typedef struct { int rank, n; ncclComm_t comm; cudaStream_t stream; size_t count; double err2, ref2; int rc; } Job;

static void* allreduce_thread(void* arg) {
  Job* j = (Job*)arg;
  j->rc = 1;
  if (cudaSetDevice(j->rank) != cudaSuccess) return NULL;
  float* buf = NULL;
  float* host = (float*)malloc(j->count * sizeof(float));
  if (cudaMalloc((void**)&buf, j->count * sizeof(float)) != cudaSuccess) return NULL;
  for (size_t k = 0; k < j->count; ++k) host[k] = 0.01f * (float)((k * 7 + (size_t)j->rank * 13) % 101) - 0.5f;
  cudaMemcpy(buf, host, j->count * sizeof(float), cudaMemcpyHostToDevice);
  ncclResult_t r = ncclAllReduce(buf, buf, j->count, ncclFloat32, ncclSum, j->comm, j->stream);
  if (r != ncclSuccess) { printf("FAIL ncclAllReduce on %d -> %d (%s)\n", j->rank, r, ncclGetErrorString(r)); return NULL; }
  if (cudaStreamSynchronize(j->stream) != cudaSuccess) return NULL;
  cudaMemcpy(host, buf, j->count * sizeof(float), cudaMemcpyDeviceToHost);
  j->err2 = j->ref2 = 0.0;
  for (size_t k = 0; k < j->count; k += 97) {
    double want = 0.0;
    for (int q = 0; q < j->n; ++q) want += 0.01 * (double)((k * 7 + (size_t)q * 13) % 101) - 0.5;
    const double d = (double)host[k] - want;
    j->err2 += d * d;
    j->ref2 += want * want;
  }
  ncclResult_t async = ncclSuccess;
  if (ncclCommGetAsyncError(j->comm, &async) != ncclSuccess || async != ncclSuccess) { printf("FAIL async error %d\n", async); return NULL; }
  cudaFree(buf);
  free(host);
  j->rc = 0;
  return NULL;
}

static int allreduce_case(int n, ncclComm_t* comms, cudaStream_t* streams, size_t count) {
  pthread_t th[8];
  Job jobs[8];
  for (int i = 0; i < n; ++i) {
    jobs[i].rank = i; jobs[i].n = n; jobs[i].comm = comms[i]; jobs[i].stream = streams[i]; jobs[i].count = count;
    pthread_create(&th[i], NULL, allreduce_thread, &jobs[i]);
  }
  int bad = 0;
  double worst = 0.0;
  for (int i = 0; i < n; ++i) {
    pthread_join(th[i], NULL);
    bad |= jobs[i].rc;
    const double rel = sqrt(jobs[i].err2 / (jobs[i].ref2 > 0.0 ? jobs[i].ref2 : 1.0));
    if (rel > worst) worst = rel;
  }
  printf("allreduce count=%zu relative_rms_err=%.4g\n", count, worst);
  if (bad) return 1;
  /* exact when native; a 4-bit code with two encodes (two-shot) stays near 0.2 of the signal's rms */
  return worst <= 0.3 ? 0 : 1;
}

int main(int argc, char** argv) {
  int version = 0;
  CHECK(ncclGetVersion(&version));
  printf("version %d; error string of 5: %s\n", version, ncclGetErrorString(5));
  if (argc < 3 || strcmp(argv[1], "run") != 0) return version > 0 ? 0 : 1;
  const int n = atoi(argv[2]);
  ncclComm_t comms[8];
  cudaStream_t streams[8];
  if (n < 1 || n > 8) return 2;
  CHECK(ncclCommInitAll(comms, n, NULL));
  for (int i = 0; i < n; ++i) {
    int count = 0, rank = -1;
    CHECK(ncclCommCount(comms[i], &count));
    CHECK(ncclCommUserRank(comms[i], &rank));
    if (count != n || rank != i) { printf("FAIL comm %d reports %d/%d\n", i, rank, count); return 1; }
    CU(cudaSetDevice(i));
    CU(cudaStreamCreate(&streams[i]));
  }
  if (allreduce_case(n, comms, streams, 1024)) return 1;
  if (allreduce_case(n, comms, streams, (size_t)8 << 20)) return 1;
  /* allocation + registration + in-place broadcast */
  float* reg[8];
  void* handles[8];
  for (int i = 0; i < n; ++i) {
    CU(cudaSetDevice(i));
    CHECK(ncclMemAlloc((void**)&reg[i], 4096 * sizeof(float)));
    CHECK(ncclCommRegister(comms[i], reg[i], 4096 * sizeof(float), &handles[i]));
    CU(cudaMemset(reg[i], i == 0 ? 0x3f : 0, 4096 * sizeof(float)));
  }
  CHECK(ncclGroupStart());
  for (int i = 0; i < n; ++i) { CU(cudaSetDevice(i)); CHECK(ncclBcast(reg[i], 4096, ncclFloat32, 0, comms[i], streams[i])); }
  CHECK(ncclGroupEnd());
  for (int i = 0; i < n; ++i) {
    unsigned int word = 0;
    CU(cudaSetDevice(i));
    CU(cudaStreamSynchronize(streams[i]));
    CU(cudaMemcpy(&word, reg[i] + 4095, 4, cudaMemcpyDeviceToHost));
    if (word != 0x3f3f3f3fu) { printf("FAIL bcast on %d: %08x\n", i, word); return 1; }
    CHECK(ncclCommDeregister(comms[i], handles[i]));
    CHECK(ncclMemFree(reg[i]));
  }
  for (int i = 0; i < n; ++i) { CU(cudaSetDevice(i)); CHECK(ncclCommDestroy(comms[i])); }
  printf("ok\n");
  return 0;
}
