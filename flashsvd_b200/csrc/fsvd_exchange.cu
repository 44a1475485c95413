// Host side of the exchange regions of a tensor-parallel decode: allocation, export / import between
// the processes of a node (CUDA IPC; the imported mapping is used with plain peer loads and stores
// only), and the per-rank exchange object.  Layout and protocol: fsvd_exchange.h.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "../../include/flashsvd_b200.h"
#include "fsvd_exchange.h"
#include "fsvd_tile.h"

namespace {

int fail(int code, const char* msg) {
  fsvd_tile_set_error(code, msg);
  return code;
}
int fail_cuda(const char* what, cudaError_t e) {
  char buf[256];
  snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
  return fail(FSVD_ERR_CUDA, buf);
}

}  // namespace

extern "C" {

size_t fsvd_exchange_region_bytes(int world, int max_rows, int d) {
  if (world < 1 || world > fsvd_exch::kMaxRanks || max_rows < 1 || d < 8) return 0;
  return fsvd_exch::region_bytes(world, max_rows, d);
}

int fsvd_exchange_region_alloc(size_t bytes, void** region) {
  if (!region || bytes < (size_t)fsvd_exch::kCtrlBytes) return fail(FSVD_ERR_ARG, "region size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return fail_cuda("cudaMalloc of the exchange region", e);
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail_cuda("zero-fill of the exchange region", e);
  }
  *region = p;
  return 0;
}

int fsvd_exchange_region_free(void* region) {
  if (!region) return 0;
  const cudaError_t e = cudaFree(region);
  return e == cudaSuccess ? 0 : fail_cuda("cudaFree of the exchange region", e);
}

int fsvd_exchange_region_export(void* region, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the export handle is 64 bytes");
  if (!region || !handle) return fail(FSVD_ERR_ARG, "null argument");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, region);
  if (e != cudaSuccess) return fail_cuda("cudaIpcGetMemHandle", e);
  memcpy(handle, &h, 64);
  return 0;
}

int fsvd_exchange_region_import(const unsigned char handle[64], void** region) {
  if (!region || !handle) return fail(FSVD_ERR_ARG, "null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail_cuda("cudaIpcOpenMemHandle (peer access between the two GPUs is needed)", e);
  *region = p;
  return 0;
}

int fsvd_exchange_region_release(void* imported_region) {
  if (!imported_region) return 0;
  const cudaError_t e = cudaIpcCloseMemHandle(imported_region);
  return e == cudaSuccess ? 0 : fail_cuda("cudaIpcCloseMemHandle", e);
}

int fsvd_exchange_create(int rank, int world, void* const* regions, int max_rows, int d, void* stream,
                         fsvd_exchange** out) {
  using namespace fsvd_exch;
  if (!regions || !out) return fail(FSVD_ERR_ARG, "null argument");
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return fail(FSVD_ERR_ARG, "rank / world (at most 8 ranks)");
  if (max_rows < 1 || max_rows > 128 || d < 8 || d % 8) return fail(FSVD_ERR_ARG, "max_rows (1..128) / d (a multiple of 8)");
  for (int q = 0; q < world; ++q)
    if (!regions[q] || (reinterpret_cast<uintptr_t>(regions[q]) & 255)) return fail(FSVD_ERR_ALIGN, "exchange regions must be 256-byte aligned");
  fsvd_exchange* ex = new fsvd_exchange();
  memset(ex, 0, sizeof(*ex));
  Geom& g = ex->geom;
  for (int q = 0; q < world; ++q) g.region[q] = reinterpret_cast<unsigned long long>(regions[q]);
  g.flag_cap = flag_capacity(d);
  g.slot_bytes = slot_capacity(max_rows, d);
  g.flags_off = kCtrlBytes;
  g.slots_off = kCtrlBytes + al256((size_t)2 * world * g.flag_cap * 4);
  g.world = world;
  g.rank = rank;
  ex->max_rows = max_rows;
  ex->d = d;
  static std::atomic<unsigned long long> next_id{1};
  ex->id = next_id.fetch_add(1);
  // the first exchange has number 1 (the flags of a fresh region read 0)
  Ctrl c = {1u, 0u};
  const cudaError_t e = cudaMemcpyAsync(regions[rank], &c, sizeof(c), cudaMemcpyHostToDevice, (cudaStream_t)stream);
  cudaError_t e2 = e == cudaSuccess ? cudaStreamSynchronize((cudaStream_t)stream) : e;
  if (e2 != cudaSuccess) {
    delete ex;
    return fail_cuda("writing the control block of the exchange region", e2);
  }
  *out = ex;
  return 0;
}

int fsvd_exchange_set_trace(fsvd_exchange* ex, void* dev_ptr, size_t bytes) {
  if (!ex) return fail(FSVD_ERR_ARG, "null argument");
  if (dev_ptr && ((reinterpret_cast<uintptr_t>(dev_ptr) & 7) || bytes < 24)) return fail(FSVD_ERR_ARG, "trace buffer: 8-byte aligned, at least 24 bytes");
  ex->trace = reinterpret_cast<unsigned long long*>(dev_ptr);
  ex->trace_cap = dev_ptr ? (unsigned)(bytes / 24 > 0xffffffffull ? 0xffffffffull : bytes / 24) : 0u;
  // plans made so far do not know the buffer: a new id, so that none of them matches any more
  static std::atomic<unsigned long long> next_id{1ull << 40};
  ex->id = next_id.fetch_add(1);
  return 0;
}

int fsvd_exchange_destroy(fsvd_exchange* ex) {
  delete ex;
  return 0;
}

}  // extern "C"
