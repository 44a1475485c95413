// Exchange of partial sums between the GPUs of a tensor-parallel decode (one process per GPU).
// Internal to the library: geometry of a rank's exchange region and the device-side address helpers
// shared by the pushing GEMM epilogue and the reducing kernel (fsvd_tile.cu), and the host object
// (fsvd_exchange.cu).
//
// Every rank owns one region of device memory with the same layout, mapped into every other rank's
// process (CUDA IPC, NVLink peer access):
//
//     [control block, 256 bytes]                   local only: sequence number, done counter
//     [slots : 2 parities x world x slot_bytes  ]  slot [parity][src] = src's partial sums as 8-byte words
//
// A word carries its own flag: word [b / 2][p] of a slot = { bf16 of row b (b even), bf16 of row
// b + 1, sequence number of the exchange (32 bits) }, written with ONE 8-byte store, which the memory
// system performs as a unit.  Exchange number k (k = 1, 2, ...; parity k & 1): the GEMM that produces
// a rank's partial sums stores every finished value pair into slot [k & 1][rank] of EVERY rank's
// region (plain peer stores, its own region included) and is done: no fence, no separate flag, so
// nothing at system scope holds up the end of the kernel (a release store after the data cost 3.6 us
// median, 8 us worst, per pushing GEMM).  The reducing kernel of a rank reads the words of its OWN
// region and takes a word when its sequence number is k (polling it otherwise), adds the `world`
// slots in rank order (so every rank computes the same bits) plus the residual, and the last of its
// CTAs advances the rank's sequence number.
// Two parities suffice: a rank can push exchange k + 2 only after it has reduced k + 1, which needs
// every peer's push of k + 1, which the peer issues after its own reduction of k has completed; a
// word left from exchange k - 2 carries k - 2 and is never taken for k.
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
  unsigned long long slots_off, slot_bytes;
  int world, rank;
};

inline size_t al256(size_t x) { return (x + 255) / 256 * 256; }
inline size_t slot_capacity(int max_rows, int d) { return al256((size_t)((max_rows + 1) / 2) * d * 8); }
inline size_t region_bytes(int world, int max_rows, int d) {
  return (size_t)kCtrlBytes + (size_t)2 * world * slot_capacity(max_rows, d);
}

#ifdef __CUDACC__
// slot [parity][src] of rank dst's region, as words
__device__ __forceinline__ unsigned long long* slot_ptr(const Geom& g, int dst, unsigned parity, int src) {
  return reinterpret_cast<unsigned long long*>(g.region[dst] + g.slots_off + (size_t)(parity * g.world + src) * g.slot_bytes);
}
__device__ __forceinline__ void st_word(unsigned long long* p, unsigned pair_bits, unsigned seq) {
  const unsigned long long w = (unsigned long long)pair_bits | ((unsigned long long)seq << 32);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_word(const unsigned long long* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
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
