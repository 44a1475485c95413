// Exchange of partial sums between the GPUs of a tensor-parallel decode (one process per GPU).
// Internal to the library: geometry of a rank's exchange region and the device-side address helpers
// shared by the pushing GEMM epilogue and the reducing kernel (fsvd_tile.cu), and the host object
// (fsvd_exchange.cu).
//
// Every rank owns one region of device memory with the same layout, mapped into every other rank's
// process (CUDA IPC, NVLink peer access):
//
//     [control block, 256 bytes]                    local only: sequence number, done counter
//     [flags   : 2 parities x world x flag_cap u32] flag [parity][src][cta] = sequence number
//     [slots   : 2 parities x world x slot_bytes  ] slot [parity][src] = src's partial sums, bf16 [rows, d]
//
// Exchange number k (k = 1, 2, ...; parity k & 1): the GEMM that produces a rank's partial sums
// stores every finished tile into slot [k & 1][rank] of EVERY rank's region (plain stores, its own
// region included), and each of its CTAs then publishes flag [k & 1][rank][cta] = k in every region
// (a CTA barrier, then a store with release semantics at system scope).  The reducing kernel of a rank polls the flags of its OWN region until all
// `world` sources have posted k, adds the world slots in rank order (so every rank computes the same
// bits) plus the residual, and the last of its CTAs advances the rank's sequence number.
// Two parities suffice: a rank can push exchange k + 2 only after it has reduced k + 1, which needs
// every peer's push of k + 1, which the peer issues after its own reduction of k has completed.
//
// Every wait is bounded (clock64 budget); when it runs out the kernel records DS_PEER_TIMEOUT in
// the workspace status word and carries on with whatever the slots hold.
//
// No counterpart in the reference: it has no multi-GPU decode (it places whole layers on devices,
// runtime/cache/attn_dense_kv.py:52-58).
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace fsvd_exch {

constexpr int kMaxRanks = 8;
constexpr int kCtrlBytes = 256;
constexpr int DS_PEER_TIMEOUT = 8;   // a wait for a peer's partial sums ran out (status_detail = the rank waited for)

struct Ctrl {
  unsigned seq;    // number of the exchange in progress (starts at 1)
  unsigned done;   // CTAs of the running reduction that have finished
};

struct Geom {
  unsigned long long region[kMaxRanks];   // base of rank q's region as mapped in this process
  unsigned long long flags_off, slots_off, slot_bytes;
  unsigned flag_cap;
  int world, rank;
};

inline size_t al256(size_t x) { return (x + 255) / 256 * 256; }
inline unsigned flag_capacity(int d) { return (unsigned)((d + 127) / 128 * 8); }   // row tiles x K segments (<= 8)
inline size_t slot_capacity(int max_rows, int d) { return al256((size_t)max_rows * d * 2); }
inline size_t region_bytes(int world, int max_rows, int d) {
  return (size_t)kCtrlBytes + al256((size_t)2 * world * flag_capacity(d) * 4) + (size_t)2 * world * slot_capacity(max_rows, d);
}

#ifdef __CUDACC__
__device__ __forceinline__ unsigned* flag_ptr(const Geom& g, int dst, unsigned parity, int src, int idx) {
  return reinterpret_cast<unsigned*>(g.region[dst] + g.flags_off) + ((size_t)(parity * g.world + src) * g.flag_cap + idx);
}
__device__ __forceinline__ unsigned char* slot_ptr(const Geom& g, int dst, unsigned parity, int src) {
  return reinterpret_cast<unsigned char*>(g.region[dst] + g.slots_off + (size_t)(parity * g.world + src) * g.slot_bytes);
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
#endif

}  // namespace fsvd_exch

// host object (fsvd_exchange.cu)
struct fsvd_exchange {
  fsvd_exch::Geom geom;
  int max_rows, d;
  unsigned long long id;   // unique per created object: cached launch plans are keyed on it, not on the address alone
  unsigned long long* trace;   // optional device buffer of trace_cap records of 3 x %globaltimer (fsvd_exchange_set_trace)
  unsigned trace_cap;
};
