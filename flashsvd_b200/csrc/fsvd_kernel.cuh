// Persistent stage interpreter for single-token decode of low-rank (W = U·V) transformers.
//
// Launch geometry: one CTA per SM (cooperative launch), 7 consumer warps + 1 producer warp
// (7 issuing lanes).
//
// Box stream.  A GEMV stage is cut into units of 16 factor rows x one K segment; units go
// round-robin to the CTAs.  A unit is a row of boxes, one box = 16 rows x kBoxRowBytes.  An
// attention stage is cut into items (sequence, head group, part of the keys); an item is a row of
// boxes of cached key rows and boxes of the same value rows (AttnItem).  The boxes of all stages of
// the program, in program order, form the CTA's box sequence.  The producer warp walks that
// sequence on its own: box number q goes into ring slot q % NS with cp.async.bulk.tensor (TMA) as
// soon as the slot's previous content has been released.  Neither the factors nor the rows cached
// by earlier launches depend on this launch's activations, so the producers run ahead of the
// consumers by the whole ring, across stage boundaries: HBM keeps streaming while the consumers
// wait for each other.  Slot s is always consumed by warp s % 7 (NS is a multiple of 7) and filled
// by producer lane s % 7, so every mbarrier sees its phases in order from a single waiting thread
// or warp.
//
// Arithmetic.  bf16: a box is the A operand (16 rows) of mma.sync.m16n8k16, the staged activation
// vector the B operand with the batch as N.  A dot product does not care about the order of k, so
// lane (g, t) feeds the k-slots it owns with 8 consecutive columns: one 16-byte shared-memory load
// of factor row g, one of row g + 8 and one of activation row g.  fp32 (parity mode): the same
// loads, plain FMAs and a quad reduction by shuffles.  A warp adds its boxes of one (unit,
// operand) in registers and leaves the sum in shared memory; the sums of the warps are added in a
// fixed order and the stage's epilogue (RoPE + cache append, SiLU·up, residual, ...) runs on the
// result, so results do not depend on timing.
//
// Dataflow between stages.  Every vector that one stage produces for another travels as 8-byte
// words {fp32 value, tag}, stored with one st.relaxed.gpu and polled with ld.relaxed.gpu until the
// tag is the one of the producing stage in this launch (fsvd_stage.h).  A CTA therefore starts a
// stage as soon as the words it needs have arrived and never fences or counts arrivals.  All
// cross-CTA reads bypass L1.  The grid barrier remains for the one edge whose consumer reads a
// plain buffer (logits -> argmax) and as the builder's fallback.
//
// All waits are bounded: a wait that runs out records an error code in SyncState::status and
// the kernel carries on without waiting again, so a fault in the protocol ends in an error
// return on the host, never in a hung device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <type_traits>
#include <utility>

#include "fsvd_stage.h"

// Stage-level functions that run once per stage (input staging, attention, the producer loop).
// Inlined: as real calls they measured slower (317 against 382 tokens/s at the same source).
#ifndef FSVD_COLD
#define FSVD_COLD __forceinline__
#endif

namespace fsvd {

constexpr int kNWC = kConsumerWarps;
constexpr int kConsThreads = kNWC * 32;
constexpr int kThreads = (kNWC + kProducerWarps) * 32;

// ----------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Barrier of the consumer warps only (the producer warps never join it).
__device__ __forceinline__ void cons_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Quotient and remainder of small non-negative integers (a < 2^22, b > 0) without the long
// integer-division sequence: (a + 0.5) / b in fp32 is at least 0.5 / b away from an integer,
// further than the error of the approximate division, and one correction step covers the rest.
// The interpreter's cold paths are bound by instruction fetch, and they are full of these.
__device__ __forceinline__ int qdiv(int a, int b) {
  int q = (int)__fdividef((float)a + 0.5f, (float)b);
  const int r = a - q * b;
  q += (r >= b ? 1 : 0) - (r < 0 ? 1 : 0);
  return q;
}
__device__ __forceinline__ int qmod(int a, int b) { return a - qdiv(a, b) * b; }

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// One 2-D box of a tiled tensor map into shared memory; completion is counted on `bar`.
__device__ __forceinline__ void tma_box_2d(uint32_t dst, const void* tmap, int col, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(col), "r"(row), "r"(bar)
      : "memory");
}
// Asks L2 for the 128-byte lines of [p, p + bytes), one line per lane and round.
__device__ __forceinline__ void prefetch_l2(const void* p, int bytes, int lane) {
  const char* c = reinterpret_cast<const char*>(p);
  for (int off = lane * 128; off < bytes; off += 32 * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ----------------------------------------------------------------------------- tagged words
// {fp32 value (low half), tag (high half)}: one 64-bit access each, so value and tag are always
// seen together.  Loads and stores are relaxed at GPU scope: they are served by L2, the point
// where all SMs meet, and a word that has been seen there by one reader is seen by every later one.
typedef unsigned long long tword;
__device__ __forceinline__ tword make_tword(float v, uint32_t tag) {
  return ((tword)tag << 32) | (tword)__float_as_uint(v);
}
__device__ __forceinline__ float tw_val(tword w) { return __uint_as_float((uint32_t)w); }
__device__ __forceinline__ uint32_t tw_tag(tword w) { return (uint32_t)(w >> 32); }
__device__ __forceinline__ void st_tword(void* base, size_t i, float v, uint32_t tag) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(reinterpret_cast<tword*>(base) + i), "l"(make_tword(v, tag))
               : "memory");
}
// two consecutive words (i even: 16-byte aligned)
__device__ __forceinline__ void st_tword2(void* base, size_t i, float v0, float v1, uint32_t tag) {
  asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(reinterpret_cast<tword*>(base) + i),
               "l"(make_tword(v0, tag)), "l"(make_tword(v1, tag))
               : "memory");
}
__device__ __forceinline__ ulonglong2 ld_tword2(const void* base, size_t i) {
  ulonglong2 v;
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];"
               : "=l"(v.x), "=l"(v.y)
               : "l"(reinterpret_cast<const tword*>(base) + i));
  return v;
}
__device__ __forceinline__ bool tw_ok(const ulonglong2& v, uint32_t tag) {
  return tw_tag(v.x) == tag && tw_tag(v.y) == tag;
}

// ----------------------------------------------------------------------------- type traits
template <typename T>
struct TT;
template <>
struct TT<__nv_bfloat16> {
  static constexpr int kVec = 8;  // elements per 16-byte vector
  static __device__ __forceinline__ float rnd(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
  }
  static __device__ __forceinline__ float ld(const void* p, size_t i) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  }
  static __device__ __forceinline__ void st(void* p, size_t i, float v) {
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  }
  // two consecutive elements of a read-only array (i even)
  static __device__ __forceinline__ float2 ldg2(const void* p, size_t i) {
    const uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(p) + i));
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x << 16);
    f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16);
    f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16);
    f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16);
    f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
};
template <>
struct TT<float> {
  static constexpr int kVec = 4;
  static __device__ __forceinline__ float rnd(float v) { return v; }
  static __device__ __forceinline__ float ld(const void* p, size_t i) {
    return reinterpret_cast<const float*>(p)[i];
  }
  static __device__ __forceinline__ void st(void* p, size_t i, float v) {
    reinterpret_cast<float*>(p)[i] = v;
  }
  static __device__ __forceinline__ float2 ldg2(const void* p, size_t i) {
    return __ldg(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(p) + i));
  }
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
};
// ----------------------------------------------------------------------------- small helpers
__device__ __forceinline__ int phys_row(int rope_half, int p) {
  if (rope_half > 0) {
    const int h = qdiv(p, rope_half);
    return h * 2 * rope_half + (p - h * rope_half);
  }
  return p;
}

// Row of the KV cache that batch row b reads and writes: its own, or row 0 for all when the batch
// rows are consecutive positions of one sequence (chunked prompt pass).
__device__ __forceinline__ int cache_row(const Stage& st, int b) { return (st.flags & SF_SHARED_CACHE) ? 0 : b; }

// First unit / item of rank `r` when the assignment is rotated by `rot` over `n` ranks.
__device__ __forceinline__ int first_item(int r, int rot, int n) {
  int f = r - rot;
  if (f < 0) f += n;
  return f;
}

__device__ __forceinline__ void trace_mark(unsigned long long* trow, int k) {
  if (trow) trow[k] = gtimer();
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

// ----------------------------------------------------------------------------- waits
struct Ring {
  uint32_t full, empty;   // shared-memory addresses of the mbarrier arrays
  uint32_t data;          // shared-memory address of slot 0
  uint32_t stride;        // bytes between slots (kBoxBytes, or kQ4BoxBytes when the program has int4 stages)
  int ns;                 // slots, a multiple of kNWC (or fewer than kNWC)
};
// Cache positions seqlens[b] of the program's sequence-length array, read once per launch into
// shared memory (the array only changes in the last stage of a step).
struct PosCache {
  const int* ptr;   // the array the cached values come from
  const int* pos;   // shared memory, one entry per batch row
};
// Launch-wide constants of a CTA, kept in shared memory: the stage functions are real calls and
// read what they need from here, so nothing but a pointer is live across a call.
struct CtaConst {
  Ring ring;
  PosCache pc;
  SyncState* sync;            // where a wait that ran out is recorded
  volatile int* giveup;       // set by the first wait that ran out: nobody in the CTA waits again
  long long limit;            // budget of a wait, SM clocks
  unsigned long long tag_base;   // tag of stage i of this launch = stage_tag(tag_base, i)
  unsigned long long* trace;  // stage timeline or null
  char* xvec;                 // staged input vector
  float* red;                 // reduction scratch
  float* part;                // warps' partial sums / attention scratch
  int* xtab;                  // first input column of every (unit, operand) of the running GEMV stage
  int xstride;
  int backoff_ns;             // pause after a failed poll of tagged words
  int gate;                   // 1: a thread polls one sample of its words before it asks for all of them
  int cap;                    // boxes in flight per producer lane (0 = ring depth)
};
// What a bounded wait needs: the CTA's constants and the stage it runs in.
struct Waiter {
  const CtaConst* cc;
  int stage;
};
struct Spin {
  long long c0;
  unsigned n;
  __device__ __forceinline__ Spin() : c0(0), n(0) {}
};
// Called after a failed poll.  False: stop waiting (the budget ran out, now or earlier).
// (A real call: it sits behind every poll of the kernel and only runs when a poll failed.)
static __device__ __noinline__ bool spin_again(const Waiter& w, Spin& sp, int code) {
  const CtaConst& cc = *w.cc;
  if (sp.n == 0) {
    if (*cc.giveup) return false;
    sp.c0 = clock64();
  }
  if (code == DS_TAG_TIMEOUT && cc.backoff_ns > 0) __nanosleep(cc.backoff_ns);
  if ((++sp.n & 31u) == 0) {
    if (*cc.giveup) return false;
    if (clock64() - sp.c0 > cc.limit) {
      if (atomicCAS(&cc.sync->status, (int)DS_OK, code) == (int)DS_OK) cc.sync->status_detail = w.stage;
      *cc.giveup = 1;
      return false;
    }
  }
  return true;
}

// Grid barrier wait (one polling lane per CTA) in front of a stage with SF_BARRIER.
__device__ __forceinline__ void barrier_wait(const Waiter& w, unsigned long long target, int tid) {
  if (tid == 0) {
    Spin sp;
    while (ld_acquire_u64(&w.cc->sync->arrivals) < target)
      if (!spin_again(w, sp, DS_BARRIER_TIMEOUT)) break;
  }
  cons_sync();
}

// Bounded wait on a ring mbarrier.  False: the wait ran out (recorded in SyncState::status) or
// this CTA has already given up; the caller goes on without the data.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const Waiter& w) {
  if (mbar_try_wait(bar, parity)) return true;
  Spin sp;
  while (!mbar_try_wait(bar, parity))
    if (!spin_again(w, sp, DS_COPY_TIMEOUT)) return false;
  return true;
}

// ----------------------------------------------------------------------------- GEMV epilogue
// Operands of an item's epilogue that do not depend on the accumulators; fetched before the
// item's boxes are consumed so that their latency hides behind them (after the stage's input has
// arrived: a residual is complete by then, see SF_RESID_TAG).  They stay raw bits until the
// epilogue: converting a loaded bf16 to float right away would stall the warp on the load.
struct EpiAux {
  unsigned r0, r1;   // raw operand bits: element of type T (bf16 in the low half) or fp32
  int pos;
};
template <typename T>
__device__ __forceinline__ unsigned raw_ld(const void* p, size_t i);
template <>
__device__ __forceinline__ unsigned raw_ld<__nv_bfloat16>(const void* p, size_t i) {
  return (unsigned)__ldcg(reinterpret_cast<const unsigned short*>(p) + i);
}
template <>
__device__ __forceinline__ unsigned raw_ld<float>(const void* p, size_t i) {
  return __ldcg(reinterpret_cast<const unsigned*>(p) + i);
}
template <typename T>
__device__ __forceinline__ float raw_to_float(unsigned r) {
  return sizeof(T) == 2 ? __uint_as_float(r << 16) : __uint_as_float(r);
}
__device__ __forceinline__ int cached_pos(const PosCache& pc, const int* seqlens, int b) {
  return seqlens == pc.ptr ? pc.pos[b] : seqlens[b];
}

template <typename T>
__device__ __forceinline__ void epi_prefetch(const Stage& st, int p, int b, EpiAux& ax, const PosCache pc) {
  ax.r0 = ax.r1 = 0u;
  ax.pos = 0;
  switch (st.epi) {
    case EPI_RESID: {
      const size_t i = (size_t)b * st.P + p;
      if (st.flags & SF_RESID_TAG) ax.r0 = raw_ld<float>(st.resid, 2 * i);   // the value half of the word
      else if (st.flags & SF_RESID_T) ax.r0 = raw_ld<T>(st.resid, i);
      else ax.r0 = raw_ld<float>(st.resid, i);
    } break;
    case EPI_ROPE_Q:
    case EPI_ROPE_K:
    case EPI_QKV: {
      const int half = st.rope_half;
      ax.pos = cached_pos(pc, st.seqlens, b);
      if (st.epi != EPI_QKV || p < (st.H + st.Hk) * half) {   // q and k rows rotate
        const int j = qmod(p, half);
        const int pt = min(ax.pos, st.S_max - 1);   // a position past the tables is reported, not read
        ax.r0 = raw_ld<T>(st.cos_tab, (size_t)pt * half + j);
        ax.r1 = raw_ld<T>(st.sin_tab, (size_t)pt * half + j);
      }
    } break;
    case EPI_V:
      ax.pos = cached_pos(pc, st.seqlens, b);
      break;
    default:
      break;
  }
}

// A plain (T or fp32) or tagged store of one output element.
template <typename T>
__device__ __forceinline__ void out_store(const Stage& st, void* out, size_t i, float v, uint32_t tag) {
  if (st.flags & SF_TAG_OUT) st_tword(out, i, v, tag);
  else if (st.flags & SF_OUT_T) TT<T>::st(out, i, v);
  else reinterpret_cast<float*>(out)[i] = v;
}

template <typename T>
__device__ __forceinline__ void gemv_epilogue(const Stage& st, int p, int b, int seg, float a, float bsum,
                                              const EpiAux& ax, uint32_t tag, SyncState* sync) {
  using X = TT<T>;
  const int P = st.P, epi = st.epi;
  if (epi == EPI_PARTIAL) {
    st_tword(st.out, ((size_t)seg * st.B + b) * P + p, a, tag);
    return;
  }
  float v = X::rnd(a);
  if (epi <= EPI_SWIGLU) {   // one value for out[b, p]
    if (epi == EPI_RESID) {
      const float res = (st.flags & SF_RESID_T) ? raw_to_float<T>(ax.r0) : __uint_as_float(ax.r0);
      v = X::rnd(res + v);
    } else if (epi == EPI_SWIGLU) {
      const float sg = X::rnd(v / (1.0f + expf(-v)));
      v = X::rnd(sg * X::rnd(bsum));
    }
    out_store<T>(st, st.out, (size_t)b * P + p, v, tag);
    return;
  }
  // Head stages.  hh = head over [q heads | k heads | v heads]; a rotary row carries two values, dims
  // (j, j + half) of its head; a row of the separate value lift carries one, dim j.
  const bool one = epi == EPI_V;
  const int half = one ? st.Dh : st.rope_half, pos = ax.pos;
  int hh = qdiv(p, half);
  const int j = p - hh * half;
  if (epi == EPI_ROPE_K) hh += st.H;
  else if (one) hh += st.H + st.Hk;
  float v2 = X::rnd(bsum);
  const bool isk = hh < st.H + st.Hk;   // q and k heads rotate
  if (isk) {
    const float c = raw_to_float<T>(ax.r0), sn = raw_to_float<T>(ax.r1);
    const float o1 = X::rnd(X::rnd(v * c) - X::rnd(v2 * sn));
    v2 = X::rnd(X::rnd(v2 * c) + X::rnd(v * sn));
    v = o1;
  }
  if (hh < st.H) {
    const size_t base = ((size_t)b * st.H + hh) * st.Dh + j;
    out_store<T>(st, st.out, base, v, tag);
    out_store<T>(st, st.out, base + half, v2, tag);
    return;
  }
  const int hk = hh - st.H - (isk ? 0 : st.Hk);
  void* const cache = (isk || one) ? st.cache : const_cast<void*>(st.vcache);
  void* const nw = isk ? st.knew : st.vnew;
  if (pos < st.S_max) {
    const size_t base = (((size_t)cache_row(st, b) * st.S_max + pos) * st.Hk + hk) * st.Dh + j;
    X::st(cache, base, v);
    if (!one) X::st(cache, base + half, v2);
  } else {
    atomicCAS(&sync->status, (int)DS_OK, (int)DS_CACHE_FULL);
  }
  if (nw) {
    const size_t nb = ((size_t)b * st.Hk + hk) * st.Dh + j;
    st_tword(nw, nb, v, tag);
    if (!one) st_tword(nw, nb + half, v2, tag);
  }
}

// ----------------------------------------------------------------------------- vector stage-in
template <typename T>
__device__ __forceinline__ void st4(char* xvec, size_t i, float4 v);
template <>
__device__ __forceinline__ void st4<float>(char* xvec, size_t i, float4 v) {
  *reinterpret_cast<float4*>(xvec + i * 4) = v;
}
template <>
__device__ __forceinline__ void st4<__nv_bfloat16>(char* xvec, size_t i, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(xvec + i * 2) = u;
}
template <typename T>
__device__ __forceinline__ void st2(char* xvec, size_t i, float a, float b);
template <>
__device__ __forceinline__ void st2<float>(char* xvec, size_t i, float a, float b) {
  *reinterpret_cast<float2*>(xvec + i * 4) = make_float2(a, b);
}
template <>
__device__ __forceinline__ void st2<__nv_bfloat16>(char* xvec, size_t i, float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  *reinterpret_cast<__nv_bfloat162*>(xvec + i * 2) = v;
}

// 16 raw bytes of a T array (8 bf16 / 4 fp32) at element index i, served by L2.
template <typename T>
__device__ __forceinline__ uint4 ld_raw16(const void* base, size_t i) {
  return __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(base) + i));
}

// Sum of the nseg tagged partial vectors [nseg][B][len], columns [col0, col0 + lenS), rounded to T.
// Per batch row a thread owns up to UP positions of two words; it walks the partial vectors in
// segment order (a fixed summation order), SG vectors per round, and per round issues the loads of
// all its positions before looking at a tag, repeating them until every word carries `tag`.
// UP x SG = 8 loads of 16 bytes in flight: every further round is another round trip to L2 on the
// critical path, more loads in flight cost registers the interpreter does not have.
template <typename T, int UP, int SG>
__device__ __forceinline__ void stage_sum_tagged(const Stage& st, char* xvec, int xstride, int col0, int lenS,
                                                 int tid, uint32_t tag, const Waiter& w) {
  constexpr int NT = kConsThreads;
  const int B = st.B, len = st.vl_len, nseg = st.vl_nseg;
  const int upr = lenS >> 1;
  const size_t segstride = (size_t)B * len;
#pragma unroll 1
  for (int b = 0; b < B; ++b) {
#pragma unroll 1
    for (int u0 = tid; u0 < upr; u0 += NT * UP) {
      const tword* base = reinterpret_cast<const tword*>(st.vl_src) + (size_t)b * len + col0 + u0 * 2;
      float a0[UP], a1[UP];
#pragma unroll
      for (int k = 0; k < UP; ++k) a0[k] = a1[k] = 0.f;
#pragma unroll 1
      for (int q = 0; q < nseg; q += SG, base += SG * segstride) {
        ulonglong2 v[SG][UP];
        Spin sp;
        for (;;) {
          bool ok = true;
#pragma unroll
          for (int g = 0; g < SG; ++g) {
            // (a round past the last vector repeats the round's first one and is not added)
            const tword* bg = base + (q + g < nseg ? g : 0) * segstride;
#pragma unroll
            for (int k = 0; k < UP; ++k)
              if (u0 + k * NT < upr) v[g][k] = ld_tword2(bg, (size_t)(k * NT * 2));
          }
#pragma unroll
          for (int g = 0; g < SG; ++g)
#pragma unroll
            for (int k = 0; k < UP; ++k)
              if (u0 + k * NT < upr) ok = ok & tw_ok(v[g][k], tag);
          if (ok || !spin_again(w, sp, DS_TAG_TIMEOUT)) break;
        }
#pragma unroll
        for (int g = 0; g < SG; ++g)
          if (q + g < nseg) {
#pragma unroll
            for (int k = 0; k < UP; ++k) {
              a0[k] += tw_val(v[g][k].x);
              a1[k] += tw_val(v[g][k].y);
            }
          }
      }
#pragma unroll
      for (int k = 0; k < UP; ++k)
        if (u0 + k * NT < upr) st2<T>(xvec, (size_t)b * xstride + (size_t)(u0 + k * NT) * 2, a0[k], a1[k]);
    }
  }
}

// Merge of the nsplit part records of one head at dims (dim, dim + 1) of batch row b (VL_ATTN and
// ST_ATTN_OUT): polls the records until they carry `tag`, then combines them in part order.
// A real call with rolled loops: it runs a handful of times per stage.
static __device__ __noinline__ float2 attn_merge2(const Stage& st, int b, int h, int dim, uint32_t tag, const Waiter& w) {
  const int cph = st.nsplit;   // <= 4
  const size_t rec0 = ((size_t)b * st.H + h) * cph;
  ulonglong2 a[4], ml[4];
  Spin sp;
  for (;;) {
    bool ok = true;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const size_t r = rec0 + (c < cph ? c : 0);   // (unused slots repeat part 0: no branches around the loads)
      a[c] = ld_tword2(st.part_acc, r * st.Dh + dim);
      ml[c] = ld_tword2(st.part_ml, r * 2);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) ok = ok & tw_ok(a[c], tag) & tw_ok(ml[c], tag);
    if (ok || !spin_again(w, sp, DS_TAG_TIMEOUT)) break;
  }
  float M = -INFINITY;
#pragma unroll
  for (int c = 0; c < 4; ++c) M = fmaxf(M, tw_val(ml[c].x));
  float L = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float lc = c < cph ? tw_val(ml[c].y) : 0.f;
    const float wgt = lc > 0.f ? expf(tw_val(ml[c].x) - M) : 0.f;
    L += lc * wgt;
    o0 = fmaf(tw_val(a[c].x), wgt, o0);
    o1 = fmaf(tw_val(a[c].y), wgt, o1);
  }
  const float invL = L > 0.f ? 1.f / L : 0.f;
  return make_float2(o0 * invL, o1 * invL);
}

// Brings the stage's input vector into shared memory as T.  Tagged sources are polled (no grid
// barrier in front of the stage); plain sources are inputs of the call.  All loads of a pass are
// issued before the first use so that their L2 latencies overlap.
template <typename T>
__device__ FSVD_COLD void stage_vector(const Stage& st, char* xvec, int xstride, float* red, float* scratch,
                                       int tid, int nthreads, uint32_t tag, const Waiter& w,
                                       unsigned long long* trow) {
  using X = TT<T>;
  constexpr int VEC = X::kVec;  // elements per 16 bytes of T
  const int len = st.vl_len, B = st.B;
  const bool tagged = (st.flags & SF_TAG_IN) != 0;
  // with SF_SEG_X only the K segment of this CTA is staged, at offset 0
  int col0 = 0, lenS = len;
  if (st.flags & SF_SEG_X) {
    const int grid = gridDim.x;
    const int seg = qmod(first_item(blockIdx.x, qmod(st.rot, grid), grid), st.segs);
    col0 = seg * st.kseg;
    lenS = len - col0 < st.kseg ? len - col0 : st.kseg;
    if (lenS < 0) lenS = 0;
  }
  if (st.vl_mode == VL_ATTN) {
    // merged attention output of columns [col0, col0 + lenS): two dims per thread and pass
    const int upr = lenS >> 1, units = B * upr;
#pragma unroll 1
    for (int u = tid; u < units; u += nthreads) {
      const int b = qdiv(u, upr), e = col0 + (u - b * upr) * 2;
      const int h = qdiv(e, st.Dh);
      const float2 o = attn_merge2(st, b, h, e - h * st.Dh, tag, w);
      st2<T>(xvec, (size_t)b * xstride + (e - col0), o.x, o.y);
    }
  } else if (st.vl_mode == VL_SUM && tagged) {
    // short vectors in several parts: 4 positions x 2 partial vectors per round; else 8 x 1
    if (st.vl_nseg > 1 && (lenS >> 1) <= kConsThreads * 4) stage_sum_tagged<T, 4, 2>(st, xvec, xstride, col0, lenS, tid, tag, w);
    else stage_sum_tagged<T, 8, 1>(st, xvec, xstride, col0, lenS, tid, tag, w);
  } else if (st.vl_mode == VL_SUM) {
    // plain T -> T copy of an input of the call
    const int upr = lenS / VEC, units = B * upr;
    for (int u = tid; u < units; u += nthreads) {
      const int b = qdiv(u, upr), k = (u - b * upr) * VEC;
      *reinterpret_cast<uint4*>(xvec + ((size_t)b * xstride + k) * sizeof(T)) =
          ld_raw16<T>(st.vl_src, (size_t)b * len + col0 + k);
    }
  } else if (st.vl_mode == VL_RMSNORM && tagged) {
    // tagged source: a thread keeps up to U positions of two words; a longer row is read twice
    constexpr int U = 10, NT = kConsThreads;
    const int warp = tid >> 5, lane = tid & 31;
    const int upr = len >> 1;
    const bool fits = upr <= NT * U;
    // the weights of this thread's positions, asked for before the wait (they do not depend on it)
    float2 wg[U];
    if (fits) {
#pragma unroll
      for (int q = 0; q < U; ++q)
        if (tid + q * NT < upr) wg[q] = X::ldg2(st.vl_w, (size_t)(tid + q * NT) * 2);
    }
#pragma unroll 1
    for (int b = 0; b < B; ++b) {
      ulonglong2 v[U];
      float ss = 0.f;
      const tword* row = reinterpret_cast<const tword*>(st.vl_src) + (size_t)b * len + tid * 2;
#pragma unroll 1
      for (int u0 = tid; u0 < upr; u0 += NT * U, row += NT * U * 2) {
        Spin sp;
        for (;;) {
          bool ok = true;
#pragma unroll
          for (int q = 0; q < U; ++q)
            if (u0 + q * NT < upr) v[q] = ld_tword2(row, (size_t)(q * NT * 2));
#pragma unroll
          for (int q = 0; q < U; ++q)
            if (u0 + q * NT < upr) ok = ok & tw_ok(v[q], tag);
          if (ok || !spin_again(w, sp, DS_TAG_TIMEOUT)) break;
        }
#pragma unroll
        for (int q = 0; q < U; ++q)
          if (u0 + q * NT < upr) {
            const float f0 = tw_val(v[q].x), f1 = tw_val(v[q].y);
            ss = fmaf(f0, f0, fmaf(f1, f1, ss));
          }
      }
      trace_mark(trow, 4);
      ss = warp_sum(ss);
      float* const rb = red + (b & 1) * 8;   // two sets of warp sums: one CTA barrier per row is enough
      if (lane == 0) rb[warp] = ss;
      cons_sync();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < kNWC; ++i) tot += rb[i];
      const float inv = rsqrtf(tot / (float)len + st.eps);
      trace_mark(trow, 5);
      if (fits) {
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = tid + q * NT;
          if (u < upr)
            st2<T>(xvec, (size_t)b * xstride + (size_t)u * 2, wg[q].x * X::rnd(tw_val(v[q].x) * inv),
                   wg[q].y * X::rnd(tw_val(v[q].y) * inv));
        }
      } else {
        // second pass over the row (its words are known to be there): U positions per round trip
        row = reinterpret_cast<const tword*>(st.vl_src) + (size_t)b * len + tid * 2;
#pragma unroll 1
        for (int u0 = tid; u0 < upr; u0 += NT * U, row += NT * U * 2) {
#pragma unroll
          for (int q = 0; q < U; ++q)
            if (u0 + q * NT < upr) {
              v[q] = ld_tword2(row, (size_t)(q * NT * 2));
              wg[q] = X::ldg2(st.vl_w, (size_t)(u0 + q * NT) * 2);
            }
#pragma unroll
          for (int q = 0; q < U; ++q) {
            const int u = u0 + q * NT;
            if (u < upr)
              st2<T>(xvec, (size_t)b * xstride + (size_t)u * 2, wg[q].x * X::rnd(tw_val(v[q].x) * inv),
                     wg[q].y * X::rnd(tw_val(v[q].y) * inv));
          }
        }
      }
    }
  } else if (st.vl_mode == VL_RMSNORM) {
    // plain T source (an input of the call), weight of type T; a row longer than the register
    // window is read twice
    constexpr int U = 3;
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    const int upr = len / VEC;
    const bool fits = upr <= nthreads * U;
    for (int b = 0; b < B; ++b) {
      uint4 v[U], wv[U];
      float ss = 0.f;
      for (int u0 = tid; u0 < upr; u0 += nthreads * U) {
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = u0 + q * nthreads;
          if (u < upr) {
            v[q] = ld_raw16<T>(st.vl_src, (size_t)b * len + (size_t)u * VEC);
            wv[q] = ld_raw16<T>(st.vl_w, (size_t)u * VEC);
          }
        }
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = u0 + q * nthreads;
          if (u < upr) {
            float f[VEC];
            X::unpack(v[q], f);
#pragma unroll
            for (int e = 0; e < VEC; ++e) ss = fmaf(f[e], f[e], ss);
          }
        }
      }
      trace_mark(trow, 4);
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      cons_sync();
      float tot = 0.f;
      for (int i = 0; i < nwarps; ++i) tot += red[i];
      const float inv = rsqrtf(tot / (float)len + st.eps);
      cons_sync();
      trace_mark(trow, 5);
      auto finish = [&](int u, const uint4& xr, const uint4& wr) {
        float f[VEC], g[VEC];
        X::unpack(xr, f);
        X::unpack(wr, g);
#pragma unroll
        for (int e = 0; e < VEC; e += 4)
          st4<T>(xvec, (size_t)b * xstride + (size_t)u * VEC + e,
                 make_float4(g[e] * X::rnd(f[e] * inv), g[e + 1] * X::rnd(f[e + 1] * inv),
                             g[e + 2] * X::rnd(f[e + 2] * inv), g[e + 3] * X::rnd(f[e + 3] * inv)));
      };
      if (fits) {
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = tid + q * nthreads;
          if (u < upr) finish(u, v[q], wv[q]);
        }
      } else {
        for (int u = tid; u < upr; u += nthreads)
          finish(u, ld_raw16<T>(st.vl_src, (size_t)b * len + (size_t)u * VEC),
                 ld_raw16<T>(st.vl_w, (size_t)u * VEC));
      }
    }
  }
}

// ----------------------------------------------------------------------------- box plans
// This CTA's share of a GEMV stage.  Unit j of the CTA is global unit first + j * grid =
// (row group, K segment); its boxes are ordered operand-major, then by column chunk.
struct BoxPlan {
  int first, nu;   // first global unit, number of units of this CTA
  int nops, cps;   // operands per unit, boxes per (unit, operand)
  int nbox;        // nu * nops * cps
};
__device__ __forceinline__ BoxPlan plan_boxes(int P, int segs, int cps, int rot, bool two_ops, int cta, int grid) {
  BoxPlan bp;
  const int total = ((P + kUnitRows - 1) / kUnitRows) * segs;
  bp.first = first_item(cta, qmod(rot, grid), grid);
  bp.nu = bp.first < total ? qdiv(total - bp.first + grid - 1, grid) : 0;
  bp.nops = two_ops ? 2 : 1;
  bp.cps = cps;
  bp.nbox = bp.nu * bp.nops * cps;
  return bp;
}

// The fields of an ST_ATTN stage that fix its items and boxes.
// A head group = GI query heads that share one kv head (GI = 1, or 2 when H/Hk is even); its keys
// are cut into cph parts, one item = (batch row, head group, part) = one CTA's work.
struct AttnP {
  int B, H, Hk, Dh, S_max, cph, rbmax, seqlen_add, GI, R, Hg, nslice, step;
  bool shared, fresh;
  const int* seqlens;
};
__device__ __forceinline__ AttnP attn_params(const Stage& st, int ring_slots) {
  AttnP ap;
  ap.B = st.B; ap.H = st.H; ap.Hk = st.Hk; ap.Dh = st.Dh; ap.S_max = st.S_max;
  ap.cph = st.nsplit; ap.rbmax = st.attn_rb; ap.seqlen_add = st.seqlen_add;
  const int G = qdiv(st.H, st.Hk);
  ap.GI = (G & 1) ? 1 : 2;
  ap.R = G / ap.GI;
  ap.Hg = st.Hk * ap.R;
  ap.nslice = st.B * ap.Hg * ap.cph;
  ap.step = ring_slots < kNWC ? ring_slots : kNWC;
  ap.shared = (st.flags & SF_SHARED_CACHE) != 0;
  ap.fresh = st.knew != nullptr;
  ap.seqlens = st.seqlens;
  return ap;
}
// Item hs: rows [j0, j1) of the cache (written by earlier launches) come through the ring; nfresh
// rows written by this launch come from the tagged side buffers (the last part takes them).  A
// batch row of a prompt chunk (shared cache) sees the chunk's rows up to its own.
// The rows of an item are cut into nch chunks of rpc rows; a chunk is kb <= 7 boxes of rb key rows
// followed by the kb boxes of the same value rows, and warp i of the CTA takes key box i and value
// box i of every chunk (in the order of the box sequence, as the ring requires).  Every box is
// fetched with rbmax rows (the tensor map's box); the rows past rb belong to the next box.
struct AttnItem {
  int b, hg, hk, part, j0, j1, nfresh, row0;
  int nch, rpc, rb, kb, kbl, nb;   // chunks, rows per chunk, rows per box, boxes per chunk, of the last chunk, all boxes
};
__device__ __forceinline__ void attn_item(const AttnP& ap, int hs, const PosCache& pc, AttnItem& it) {
  const int hq = qdiv(hs, ap.cph);
  it.part = hs - hq * ap.cph;
  it.b = qdiv(hq, ap.Hg);
  it.hg = hq - it.b * ap.Hg;
  it.hk = qdiv(it.hg, ap.R);
  const int n = min(cached_pos(pc, ap.seqlens, it.b) + ap.seqlen_add, ap.S_max);
  it.nfresh = ap.fresh ? min(n, ap.shared ? it.b + 1 : 1) : 0;
  const int n_old = n - it.nfresh;
  const int per = qdiv(n_old + ap.cph - 1, ap.cph);
  it.j0 = min(n_old, it.part * per);
  it.j1 = min(n_old, it.j0 + per);
  it.row0 = (ap.shared ? 0 : it.b) * ap.S_max + it.j0;
  const int len = it.j1 - it.j0;
  if (len <= 0) {
    it.nch = it.rpc = it.kb = it.kbl = it.nb = 0;
    it.rb = 1;
    return;
  }
  const int cap = ap.step * ap.rbmax;
  it.nch = qdiv(len + cap - 1, cap);
  it.rpc = qdiv(len + it.nch - 1, it.nch);
  it.rb = qdiv(it.rpc + ap.step - 1, ap.step);
  it.kb = qdiv(it.rpc + it.rb - 1, it.rb);
  const int last = len - (it.nch - 1) * it.rpc;
  it.kbl = qdiv(last + it.rb - 1, it.rb);
  it.nb = 2 * ((it.nch - 1) * it.kb + it.kbl);
}

// ----------------------------------------------------------------------------- producer
// The producer warp.  Lane L < N (N = 7, or the slot count of a smaller ring) owns the boxes
// q with q % N == L, which always land in the slots s with s % N == L: a lane waits only on the
// mbarriers of its own slots and sees their phases in order (a parity wait cannot tell phase k
// from phase k + 2).  The lanes walk the CTA's box sequence of the whole program in lockstep, N
// boxes per round: every lane keeps its own cursor, waits for its slot, and then all lanes issue
// their TMA copies with one instruction.  (Lanes that ran their own loops and met at different
// barriers serialised: 1 such lane gave 354, 4 lanes 327, 8 lanes 298 tokens/s on the 7B-shape
// model; 7 lanes in lockstep 368.)
template <typename T, bool Q4>
__device__ FSVD_COLD void producer_loop(const Stage* prog, int nstages, const unsigned char* maps,
                                        const CtaConst& cc, int lane) {
  const Ring rg = cc.ring;
  Waiter w = {&cc, 0};
  constexpr int BOXCOLS = kBoxRowBytes / (int)sizeof(T);
  const int grid = gridDim.x, cta = blockIdx.x;
  const int N = rg.ns < kNWC ? rg.ns : kNWC;
  const unsigned mask = (1u << N) - 1u;
  if (lane >= N) return;
  // Cursor: stage s, box l of the current run of `lim` boxes (a GEMV stage's boxes of this CTA, or
  // the boxes of one attention item).  One loop moves it; the code of a move exists once.
  int s = -1, l = 0, lim = 0;
  bool done = false, attn = false;
  int nops = 1, cps = 1, first = 0, segs = 1, half = 0;
  int nch = 0;                               // > 0: the stage streams int4 tiles, nch per tile row
  AttnP ap = {};
  AttnItem ai = {};
  int hs = 0;
  const unsigned char* mapA = maps;
  int slot = lane, round = 0, issue = 0;
  // cap > 0: at most `cap` boxes of a lane are in flight (issued and not yet landed)
  const int spl = rg.ns / N;   // slots per lane
  const int cap = cc.cap >= spl ? 0 : cc.cap;
  int k = lane;   // boxes to move before the next issue
  for (;;) {
    l += k;
#pragma unroll 1
    while (!done && l >= lim) {
      l -= lim;
      lim = 0;
      if (attn && (hs += grid) < ap.nslice) {
        attn_item(ap, hs, cc.pc, ai);
        lim = ai.nb;
        continue;
      }
      attn = false;
      if (++s >= nstages) {
        done = true;
        break;
      }
      const Stage& st = prog[s];
      mapA = maps + (size_t)(2 * s) * 128;
      if (st.type == ST_GEMV) {
        const BoxPlan bp = plan_boxes(st.P, st.segs, st.cps, st.rot, st.WB != nullptr, cta, grid);
        nops = bp.nops; cps = bp.cps; first = bp.first; segs = st.segs; half = st.rope_half;
        nch = (Q4 && (st.flags & SF_Q4)) ? st.nch : 0;
        lim = bp.nbox;
      } else if (st.type == ST_ATTN) {
        ap = attn_params(st, rg.ns);
        hs = first_item(cta, qmod(st.rot, grid), grid) - grid;   // the loop steps to the first item
        attn = true;
      }
    }
    if (!__any_sync(mask, !done)) break;
    bool ok = !done;
    w.stage = s;
    if (ok && cap > 0 && issue >= cap) {
      const int pi = issue - cap;
      const int pr = pi / spl, ps = lane + N * (pi - pr * spl);
      ok = mbar_wait(rg.full + ps * 8, (uint32_t)pr & 1u, w);
    }
    if (ok && round > 0) ok = mbar_wait(rg.empty + slot * 8, (uint32_t)(round - 1) & 1u, w);
    __syncwarp(mask);
    if (ok) {
      const uint32_t fb = rg.full + slot * 8;
      const uint32_t dst = rg.data + (uint32_t)slot * (Q4 ? rg.stride : (uint32_t)kBoxBytes);
      if (attn) {
        // box l of the item: chunk c, key box i (or value box i) = rbmax rows of one kv head from
        // row i * rb of the chunk on (rows past the cache arrive as zeros)
        int c = qdiv(l, 2 * ai.kb), kbc = ai.kb;
        if (c >= ai.nch - 1) {
          c = ai.nch - 1;
          kbc = ai.kbl;
        }
        const int r = l - c * 2 * ai.kb;
        const int isv = r >= kbc ? 1 : 0;
        const int row = ai.row0 + c * ai.rpc + (r - isv * kbc) * ai.rb;
        mbar_expect_tx(fb, (uint32_t)(ap.rbmax * ap.Dh) * (uint32_t)sizeof(T));
        tma_box_2d(dst, mapA + isv * 128, ai.hk * ap.Dh, row, fb);
      } else {
        // box l of the stage: (unit ordinal, operand, chunk), unit = (row group, K segment)
        const int io = qdiv(l, cps), c = l - io * cps;
        const int j = nops == 2 ? (io >> 1) : io, op = nops == 2 ? (io & 1) : 0;
        const int uidx = first + j * grid;
        const int grp = qdiv(uidx, segs), seg = uidx - grp * segs;
        int x = (seg * cps + c) * BOXCOLS, y = phys_row(half, grp * kUnitRows);
        uint32_t bytes = kBoxBytes;
        if (Q4 && nch > 0) {
          // tile (row group, chunk) of the int4 stream; a chunk past the last tile of the row (the
          // tail of the last K segment) is fetched from outside the tensor and arrives as zeros
          // (zero scales)
          const int chunk = seg * cps + c;
          y = chunk < nch ? ((y / kUnitRows) * nch + chunk) * kQ4TileRows : 0x40000000;
          x = 0;
          bytes = kQ4BoxBytes;
        }
        mbar_expect_tx(fb, bytes);
        tma_box_2d(dst, mapA + (op ? 128 : 0), x, y, fb);
      }
    } else if (!done) {
      done = true;   // a wait ran out: this lane stops (the consumers give up on their own)
    }
    k = N;
    ++issue;
    slot += N;
    if (slot >= rg.ns) {
      slot -= rg.ns;
      ++round;
    }
  }
}

// One int4 tile (16 rows x 1024 inputs, 8 groups of 128) times the staged bf16 vector.
// wb: this lane's 16 bytes of code row g (row g + 8 is 8 rows further); sb: the tile's scale
// row; xq: the lane's 32 inputs of group 0 (64 bytes; group j is 256 bytes further).
// A warp-wide 16-byte load covers exactly one group of one row: lane t holds the codes of
// inputs 32 t .. 32 t + 31 of the group.  Word i of those 16 bytes holds inputs 8 i .. 8 i + 7,
// even inputs in the nibbles of the low half, odd inputs in the high half (fsvd_q4_pack orders
// them so): (w >> 4 n) & 0x000f000f is the pair of inputs (2 n, 2 n + 1) in the two halves of a
// register, OR 0x4300 makes each the bf16 number 128 + code, minus 136 gives code - 8 exactly.
// The pairs line up with the bf16 pairs of the staged vector, so the vector side needs no
// shuffling.  A group's 8 MMAs start from zero; the sum is scaled by the (row, group) scale in
// fp32: y = sum_groups s * sum_k (code - 8) x.
__device__ __forceinline__ uint32_t q4_pair(uint32_t w) {
  const uint32_t v = (w & 0x000f000fu) | 0x43004300u;
  const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v), __floats2bfloat162_rn(136.f, 136.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)(h & 0xffffu)));
}
__device__ __forceinline__ void q4_box(uint32_t wb, uint32_t sb, uint32_t xq, int g, float* acc) {
  const uint4 sg = lds128(sb + g * 16), sh = lds128(sb + (g + 8) * 16);
  const uint32_t sgw[4] = {sg.x, sg.y, sg.z, sg.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint4 lo = lds128(wb + j * 64), hi = lds128(wb + 8 * kQ4RowBytes + j * 64);
    const uint32_t low[4] = {lo.x, lo.y, lo.z, lo.w}, hiw[4] = {hi.x, hi.y, hi.z, hi.w};
    float ga[4] = {0.f, 0.f, 0.f, 0.f}, gb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 xv = lds128(xq + j * 256 + i * 16);
      const uint32_t wl = low[i], wh = hiw[i];
      mma_bf16_16816(ga, q4_pair(wl), q4_pair(wh), q4_pair(wl >> 4), q4_pair(wh >> 4), xv.x, xv.y);
      mma_bf16_16816(gb, q4_pair(wl >> 8), q4_pair(wh >> 8), q4_pair(wl >> 12), q4_pair(wh >> 12), xv.z, xv.w);
    }
    const float s0 = half_bits_to_float(sgw[j >> 1] >> ((j & 1) * 16));
    const float s1 = half_bits_to_float(shw[j >> 1] >> ((j & 1) * 16));
    acc[0] = fmaf(s0, ga[0] + gb[0], acc[0]);
    acc[1] = fmaf(s0, ga[1] + gb[1], acc[1]);
    acc[2] = fmaf(s1, ga[2] + gb[2], acc[2]);
    acc[3] = fmaf(s1, ga[3] + gb[3], acc[3]);
  }
}

// Timeline row of (stage s, this CTA), written by thread 0 only.
__device__ __forceinline__ unsigned long long* trace_row(const CtaConst& cc, int s) {
  return (cc.trace && threadIdx.x == 0) ? cc.trace + ((size_t)s * gridDim.x + blockIdx.x) * 16 : nullptr;
}

// ----------------------------------------------------------------------------- GEMV stage
// One GEMV stage, consumer warps.  Returns the number of boxes of this CTA in the stage.
template <typename T, bool Q4>
__device__ FSVD_COLD int gemv_stage(const Stage& st, const CtaConst& cc, int s, unsigned seq_base,
                                    unsigned long long bar_target) {
  using X = TT<T>;
  const Waiter w = {&cc, s};
  unsigned long long* const trow = trace_row(cc, s);
  constexpr int BOXCOLS = kBoxRowBytes / (int)sizeof(T);
  constexpr int NCH64 = kBoxRowBytes / 64;   // 64-byte column pieces of a box row (one per lane quad)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int B = st.B, grid = gridDim.x, segs = st.segs;
  const BoxPlan bp = plan_boxes(st.P, segs, st.cps, st.rot, st.WB != nullptr, blockIdx.x, grid);
  const int cps = bp.cps, nops = bp.nops;
  const int rowsB = kUnitRows * B;
  const bool q4 = Q4 && sizeof(T) == 2 && (st.flags & SF_Q4);
  const int boxcols = (Q4 && q4) ? kQ4BoxCols : BOXCOLS;
  const uint32_t tag_out = stage_tag(cc.tag_base, s);

  trace_mark(trow, 8);
  if (st.flags & SF_BARRIER) barrier_wait(w, bar_target, tid);
  trace_mark(trow, 1);
  // A CTA without units neither reads the stage's input nor writes anything.
  if (bp.nu == 0) return 0;
  // First input column of every (unit, operand) of this CTA, as a table in shared memory: the box
  // loop below then has no index arithmetic.  Written before the wait for the input (it does not
  // depend on it) and published by the CTA barrier behind the stage-in.
  int* const xtab = cc.xtab;
  const int nio = bp.nu * nops;   // <= kMaxUnitOps (checked by the program builder)
  for (int i = tid; i < nio; i += kConsThreads) {
    const int j = nops == 2 ? (i >> 1) : i, op = nops == 2 ? (i & 1) : 0;
    const int uidx = bp.first + j * grid;
    const int seg = qmod(uidx, segs);
    int x0 = (op ? st.xB_off : st.xA_off) + ((st.flags & SF_SEG_X) ? 0 : seg * cps * boxcols);
    if (st.epi == EPI_QKV) {   // segs == 1: uidx is the row group; the part's input starts at part * K
      const int p0 = uidx * kUnitRows, half = st.rope_half;
      x0 += ((p0 >= st.H * half) + (p0 >= (st.H + st.Hk) * half)) * st.K;
    }
    xtab[i] = x0;
  }
  // ---- wait for the words of the input vector, stage it
  if (st.vl_mode != VL_NONE) {
    stage_vector<T>(st, cc.xvec, cc.xstride, cc.red, cc.part, tid, kConsThreads, stage_tag(cc.tag_base, st.in_stage),
                    w, trow);
    cons_sync();
  }
  trace_mark(trow, 2);

  // operands of the epilogues this thread will run (outputs tid and tid + 224), fetched now so
  // that their latency hides behind the boxes
  const int nout = bp.nu * rowsB;
  auto out_pos = [&](int o, int& j, int& b, int& r, int& seg, int& p) {
    j = qdiv(o, rowsB);
    const int rem = o - j * rowsB;
    b = rem >> 4;
    r = rem & 15;
    const int uidx = bp.first + j * grid;
    const int grp = qdiv(uidx, segs);
    seg = uidx - grp * segs;
    p = grp * kUnitRows + r;
  };
  EpiAux ax0, ax1;
  ax0.r0 = ax0.r1 = ax1.r0 = ax1.r1 = 0u;
  ax0.pos = ax1.pos = 0;
  {
    int j, b, r, seg, p;
    if (tid < nout) {
      out_pos(tid, j, b, r, seg, p);
      if (p < st.P) epi_prefetch<T>(st, p, b, ax0, cc.pc);
    }
    if (tid + kConsThreads < nout) {
      out_pos(tid + kConsThreads, j, b, r, seg, p);
      if (p < st.P) epi_prefetch<T>(st, p, b, ax1, cc.pc);
    }
  }

  // ---- this warp's boxes: local box l belongs to warp (seq_base + l) % step
  const int g = lane >> 2, t = lane & 3;
  const uint32_t xrow_bytes = (uint32_t)cc.xstride * (uint32_t)sizeof(T);
  const uint32_t xvec_s = smem_u32(cc.xvec) + t * 16;
  const uint32_t xlane_s = xvec_s + (uint32_t)(g < B ? g : 0) * xrow_bytes;
  const uint32_t wlane = (uint32_t)g * ((Q4 && q4) ? kQ4RowBytes : kBoxRowBytes) + t * 16;
  // Box number q is consumed by warp q % step: step = 7 for a ring of 7, 14 or 21 slots; a ring
  // of fewer than 7 slots (huge input vectors) has one warp per slot and leaves the others idle.
  const int step = cc.ring.ns < kNWC ? cc.ring.ns : kNWC;
  const int KK = cps < step ? cps : step;   // warps that hold partial sums of one (unit, operand)
  int l = warp < step ? qmod(warp - qmod((int)seq_base, step) + step, step) : bp.nbox;
  int slot, round;
  {
    const unsigned seq0 = seq_base + (unsigned)l;
    round = qdiv((int)seq0, cc.ring.ns);
    slot = (int)(seq0 - (unsigned)round * cc.ring.ns);
  }
  int io = qdiv(l, cps), c = l - io * cps;   // (unit ordinal * nops + operand), chunk inside it
  int cur_io = -1, cur_kk = 0, xcol0 = 0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};          // bf16: mma accumulators (rows g, g+8; batch 2t, 2t+1)
  float accf[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // fp32: [row half][batch]
  auto flush = [&]() {
    float* dst = cc.part + ((size_t)cur_io * KK + cur_kk) * rowsB;
    if constexpr (sizeof(T) == 2) {
      if (2 * t < B) {
        dst[(2 * t) * 16 + g] = acc[0];
        dst[(2 * t) * 16 + g + 8] = acc[2];
      }
      if (2 * t + 1 < B) {
        dst[(2 * t + 1) * 16 + g] = acc[1];
        dst[(2 * t + 1) * 16 + g + 8] = acc[3];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] = 0.f;
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) {
          float v = accf[h][bb];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if (t == 0 && bb < B) dst[bb * 16 + g + 8 * h] = v;
          accf[h][bb] = 0.f;
        }
    }
  };
  for (; l < bp.nbox; l += step) {
    if (io != cur_io) {
      if (cur_io >= 0) flush();
      cur_io = io;
      cur_kk = c;   // the first chunk of a warp in a (unit, operand) is below step
      xcol0 = xtab[io];
    }
    bool ok = mbar_wait(cc.ring.full + slot * 8, (uint32_t)round & 1u, w);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const uint32_t wb = cc.ring.data + (uint32_t)slot * (Q4 ? cc.ring.stride : (uint32_t)kBoxBytes) + wlane;
      const uint32_t xoff = (uint32_t)(xcol0 + c * boxcols) * (uint32_t)sizeof(T);
      if constexpr (sizeof(T) == 2) {
       if (Q4 && q4) {
        q4_box(wb, wb - wlane + kUnitRows * kQ4RowBytes, xlane_s + xoff + t * 48, g, acc);
       } else {
        const uint32_t xb = xlane_s + xoff;
        // four independent accumulator chains keep the tensor pipe busy
        float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
        float a2[4] = {0.f, 0.f, 0.f, 0.f}, a3[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q + 1 < NCH64; q += 2) {
          const uint4 xv = lds128(xb + q * 64), xw = lds128(xb + q * 64 + 64);
          const uint4 lo = lds128(wb + q * 64), lp = lds128(wb + q * 64 + 64);
          const uint4 hi = lds128(wb + 8 * kBoxRowBytes + q * 64), hj = lds128(wb + 8 * kBoxRowBytes + q * 64 + 64);
          mma_bf16_16816(a0, lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
          mma_bf16_16816(a1, lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
          mma_bf16_16816(a2, lp.x, hj.x, lp.y, hj.y, xw.x, xw.y);
          mma_bf16_16816(a3, lp.z, hj.z, lp.w, hj.w, xw.z, xw.w);
        }
        if constexpr (NCH64 & 1) {
          constexpr int q = NCH64 - 1;
          const uint4 xv = lds128(xb + q * 64);
          const uint4 lo = lds128(wb + q * 64);
          const uint4 hi = lds128(wb + 8 * kBoxRowBytes + q * 64);
          mma_bf16_16816(a0, lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
          mma_bf16_16816(a1, lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) a0[e] += a2[e], a1[e] += a3[e];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] += a0[e] + a1[e];
       }
      } else {
        const uint32_t xb = xvec_s + xoff;
#pragma unroll
        for (int q = 0; q < NCH64; ++q) {
          float lo[4], hi[4], xf[4];
          X::unpack(lds128(wb + q * 64), lo);
          X::unpack(lds128(wb + 8 * kBoxRowBytes + q * 64), hi);
#pragma unroll
          for (int bb = 0; bb < 4; ++bb) {
            if (bb < B) {
              X::unpack(lds128(xb + bb * xrow_bytes + q * 64), xf);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                accf[0][bb] = fmaf(lo[e], xf[e], accf[0][bb]);
                accf[1][bb] = fmaf(hi[e], xf[e], accf[1][bb]);
              }
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(cc.ring.empty + slot * 8);
    slot += step;
    if (slot >= cc.ring.ns) {
      slot -= cc.ring.ns;
      ++round;
    }
    c += step;
    while (c >= cps) {
      c -= cps;
      ++io;
    }
  }
  if (cur_io >= 0) flush();
  trace_mark(trow, 7);
  cons_sync();
  trace_mark(trow, 10);

  // ---- add the warps' partial sums in chunk order and run the epilogue
  for (int o = tid, it = 0; o < nout; o += kConsThreads, ++it) {
    int j, b, r, seg, p;
    out_pos(o, j, b, r, seg, p);
    if (p >= st.P) continue;
    EpiAux ax;
    if (it == 0) ax = ax0;
    else if (it == 1) ax = ax1;
    else epi_prefetch<T>(st, p, b, ax, cc.pc);
    const float* src = cc.part + ((size_t)(j * nops) * KK) * rowsB + b * 16 + r;
    float sum0 = 0.f, sum1 = 0.f;
    for (int k2 = 0; k2 < KK; ++k2) sum0 += src[(size_t)k2 * rowsB];
    if (nops == 2)
      for (int k2 = 0; k2 < KK; ++k2) sum1 += src[(size_t)(KK + k2) * rowsB];
    gemv_epilogue<T>(st, p, b, seg, sum0, sum1, ax, tag_out, cc.sync);
  }
  trace_mark(trow, 11);
  return bp.nbox;
}

// ----------------------------------------------------------------------------- attention stage
// DPL consecutive elements of type T at a shared-memory address, as fp32.
template <typename T, int DPL>
__device__ __forceinline__ void lds_row(uint32_t addr, float* o);
template <>
__device__ __forceinline__ void lds_row<__nv_bfloat16, 4>(uint32_t addr, float* o) {
  const uint2 u = lds64(addr);
  o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xffff0000u);
  o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xffff0000u);
}
template <>
__device__ __forceinline__ void lds_row<__nv_bfloat16, 2>(uint32_t addr, float* o) {
  const uint32_t u = lds32(addr);
  o[0] = __uint_as_float(u << 16); o[1] = __uint_as_float(u & 0xffff0000u);
}
template <>
__device__ __forceinline__ void lds_row<float, 4>(uint32_t addr, float* o) {
  const uint4 u = lds128(addr);
  o[0] = __uint_as_float(u.x); o[1] = __uint_as_float(u.y); o[2] = __uint_as_float(u.z); o[3] = __uint_as_float(u.w);
}
template <>
__device__ __forceinline__ void lds_row<float, 2>(uint32_t addr, float* o) {
  const uint2 u = lds64(addr);
  o[0] = __uint_as_float(u.x); o[1] = __uint_as_float(u.y);
}
// DPL consecutive elements of a plain T array in global memory (an input of the call), as fp32.
template <typename T, int DPL>
__device__ __forceinline__ void ldg_row(const void* base, size_t i, float* o) {
#pragma unroll
  for (int d = 0; d < DPL; ++d) o[d] = TT<T>::ld(base, i + d);
}
// DPL consecutive tagged words, polled until they carry `tag`.
template <int DPL>
__device__ __forceinline__ void ld_tagged_row(const void* base, size_t i, uint32_t tag, const Waiter& w, float* o) {
  ulonglong2 v[DPL / 2];
  Spin sp;
  for (;;) {
    bool ok = true;
#pragma unroll
    for (int d = 0; d < DPL / 2; ++d) v[d] = ld_tword2(base, i + 2 * d);
#pragma unroll
    for (int d = 0; d < DPL / 2; ++d) ok = ok && tw_ok(v[d], tag);
    if (ok || !spin_again(w, sp, DS_TAG_TIMEOUT)) break;
  }
#pragma unroll
  for (int d = 0; d < DPL / 2; ++d) {
    o[2 * d] = tw_val(v[d].x);
    o[2 * d + 1] = tw_val(v[d].y);
  }
}

// A box of nrows cached key rows (rowb bytes apart; this lane's dims at its own offset) turned into
// probabilities against the running maximum of the warp.  Partial dot products (this lane's dims)
// go to a [key][lane] tile in shared memory; lane r then adds row r, so that every lane owns one
// full score: softmax costs one exp per lane and 2 x 5 shuffles per head instead of 5 shuffles
// and one exp per key.  Rows past nrows hold other rows of the cache or nothing defined: their
// scores are masked by selection.  Leaves the probabilities in pbuf[g * RBM + u] and rescales acc.
template <typename T, int GI, int DPL>
__device__ __forceinline__ void attn_scores(uint32_t ka, int nrows, uint32_t rowb, const float (&q)[GI][DPL],
                                            float (&acc)[GI][DPL], float (&m)[GI], float (&l)[GI], float* tile,
                                            float* pbuf, float scale, int lane) {
  constexpr int RBM = 32 / GI;
  // (rolled loops: this code runs once per stage and is bound by instruction fetch)
#pragma unroll 1
  for (int u = 0; u < nrows; u += 2) {
    float kf[2][DPL];
    lds_row<T, DPL>(ka + u * rowb, kf[0]);
    lds_row<T, DPL>(ka + (u + 1 < nrows ? u + 1 : u) * rowb, kf[1]);
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int g = 0; g < GI; ++g) {
        float s2 = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) s2 = fmaf(q[g][d], kf[r][d], s2);
        tile[(g * RBM + u + r) * 33 + lane] = s2;   // (row u + 1 of the tile may be past nrows: never read)
      }
  }
  __syncwarp();
  float sa = 0.f, sb = 0.f;
  const int gu = lane / RBM, uu = lane - gu * RBM;   // head and key of this lane's score
  const bool valid = uu < nrows;
  if (valid) {
    const float* row = tile + lane * 33;
#pragma unroll 1
    for (int i = 0; i < 32; i += 4) {
      sa += row[i] + row[i + 2];
      sb += row[i + 1] + row[i + 3];
    }
  }
  const float score = valid ? (sa + sb) * scale : -INFINITY;
  float pmine = 0.f;
#pragma unroll
  for (int g = 0; g < GI; ++g) {
    const bool mine = valid && gu == g;
    const float cm = warp_max(mine ? score : -INFINITY);
    const float mn = fmaxf(m[g], cm);
    const float corr = (m[g] == -INFINITY) ? 0.f : expf(m[g] - mn);
    const float pg = mine ? expf(score - mn) : 0.f;
    const float ls = warp_sum(pg);
    if (mine) pmine = pg;
    l[g] = l[g] * corr + ls;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[g][d] *= corr;
    m[g] = mn;
  }
  pbuf[lane] = pmine;
  __syncwarp();
}
// The box of the same nrows value rows, weighted by the probabilities attn_scores left in pbuf
// (values of rows past nrows are never multiplied).
template <typename T, int GI, int DPL>
__device__ __forceinline__ void attn_values(uint32_t va, int nrows, uint32_t rowb, float (&acc)[GI][DPL],
                                            const float* pbuf) {
  constexpr int RBM = 32 / GI;
#pragma unroll 1
  for (int u = 0; u < nrows; u += 2) {
    const bool two = u + 1 < nrows;
    float vf[2][DPL];
    lds_row<T, DPL>(va + u * rowb, vf[0]);
    lds_row<T, DPL>(va + (two ? u + 1 : u) * rowb, vf[1]);
#pragma unroll
    for (int g = 0; g < GI; ++g) {
      const float p0 = pbuf[g * RBM + u], p1 = two ? pbuf[g * RBM + u + 1] : 0.f;
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[g][d] = fmaf(p1, two ? vf[1][d] : 0.f, fmaf(p0, vf[0][d], acc[g][d]));
    }
  }
  __syncwarp();   // the tile and pbuf are rewritten by the next box
}

// Attention of the new token over the dense cache, CTA-cooperative.  Warp i of the CTA takes key
// box i and value box i of every chunk of the item (AttnItem) and folds them into a running (max,
// sum, accumulator) state per query head, lane l owning dims [l*DPL, (l+1)*DPL).  The rows that
// this launch itself appends (the new token; a prompt chunk's rows up to the batch row's own) are
// not read from the cache: the lift stages also write them as tagged words, and a warp without a
// box in the last chunk (warp 0 when there is none) polls those.  The warps' states meet in shared
// memory and are merged in warp order; the result is the item's part record, written as tagged
// words and merged with the head's other parts by whoever consumes the attention output.
// Returns the number of boxes of this CTA in the stage.
template <typename T, int GI, int DPL>
__device__ FSVD_COLD int attn_stage(const Stage& st, const CtaConst& cc, int s, unsigned seq_base) {
  const Waiter w = {&cc, s};
  unsigned long long* const trow = trace_row(cc, s);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ns = cc.ring.ns;
  const AttnP ap = attn_params(st, ns);
  const int Dh = ap.Dh, H = ap.H, grid = gridDim.x;
  const int rec = Dh + 2;                  // floats of one partial result: acc[Dh], max, sum
  float* const sh = cc.part;
  // per-warp scratch behind the partial results: score tile [33][33] and probabilities [32]
  float* const tile = sh + kNWC * GI * rec + warp * (33 * 33 + 32);
  float* const pbuf = tile + 33 * 33;
  const uint32_t rowb = (uint32_t)Dh * (uint32_t)sizeof(T);
  const uint32_t laneoff = (uint32_t)(lane * DPL) * (uint32_t)sizeof(T);
  const bool qT = (st.flags & SF_IN_T) != 0;
  const uint32_t tag_q = stage_tag(cc.tag_base, st.in_stage), tag_k = stage_tag(cc.tag_base, st.k_stage),
                 tag_v = stage_tag(cc.tag_base, st.v_stage), tag_out = stage_tag(cc.tag_base, s);
  unsigned seq = seq_base;
  int total = 0;
#pragma unroll 1
  for (int hs = first_item(blockIdx.x, qmod(st.rot, grid), grid); hs < ap.nslice; hs += grid) {
    AttnItem it;
    attn_item(ap, hs, cc.pc, it);
    float q[GI][DPL], acc[GI][DPL], m[GI], l[GI];
#pragma unroll
    for (int g = 0; g < GI; ++g) {
      const size_t qi = ((size_t)it.b * H + it.hg * GI + g) * Dh + lane * DPL;
      if (qT) ldg_row<T, DPL>(st.q, qi, q[g]);
      else ld_tagged_row<DPL>(st.q, qi, tag_q, w, q[g]);
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[g][d] = 0.f;
      m[g] = -INFINITY;
      l[g] = 0.f;
    }
    trace_mark(trow, 4);
    // ---- this warp's key box and value box of every chunk
#pragma unroll 1
    for (int c = 0; c < it.nch; ++c) {
      const int kbc = c == it.nch - 1 ? it.kbl : it.kb;
      if (warp < kbc) {
        const int rows_c = c == it.nch - 1 ? (it.j1 - it.j0) - c * it.rpc : it.rpc;
        const int nrows = min(it.rb, rows_c - warp * it.rb);
        int sq = (int)seq + c * 2 * it.kb + warp;
        int round = qdiv(sq, ns), slot = sq - round * ns;
        bool ok = mbar_wait(cc.ring.full + slot * 8, (uint32_t)round & 1u, w);
        ok = __all_sync(0xffffffffu, ok);
        trace_mark(trow, 9);
        if (ok)
          attn_scores<T, GI, DPL>(cc.ring.data + (uint32_t)slot * cc.ring.stride + laneoff, nrows, rowb, q, acc, m, l,
                                  tile, pbuf, st.scale, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(cc.ring.empty + slot * 8);
        trace_mark(trow, 12);
        sq += kbc;
        round = qdiv(sq, ns);
        slot = sq - round * ns;
        bool okv = mbar_wait(cc.ring.full + slot * 8, (uint32_t)round & 1u, w);
        okv = __all_sync(0xffffffffu, okv);
        trace_mark(trow, 13);
        if (ok && okv)
          attn_values<T, GI, DPL>(cc.ring.data + (uint32_t)slot * cc.ring.stride + laneoff, nrows, rowb, acc, pbuf);
        __syncwarp();
        if (lane == 0) mbar_arrive(cc.ring.empty + slot * 8);
      }
    }
    trace_mark(trow, 5);
    // ---- the rows this launch appends, from the tagged side buffers
    if (it.nfresh > 0 && it.part == ap.cph - 1 && warp == (it.kbl < ap.step ? it.kbl : 0)) {
#pragma unroll 1
      for (int r = 0; r < it.nfresh; ++r) {
        const int sr = ap.shared ? r : it.b;
        const size_t ki = ((size_t)sr * ap.Hk + it.hk) * Dh + lane * DPL;
        float kf[DPL], vf[DPL];
        ld_tagged_row<DPL>(st.knew, ki, tag_k, w, kf);
        ld_tagged_row<DPL>(st.vnew, ki, tag_v, w, vf);
#pragma unroll
        for (int g = 0; g < GI; ++g) {
          float s2 = 0.f;
#pragma unroll
          for (int d = 0; d < DPL; ++d) s2 = fmaf(q[g][d], kf[d], s2);
          const float score = warp_sum(s2) * st.scale;
          const float mn = fmaxf(m[g], score);
          const float corr = (m[g] == -INFINITY) ? 0.f : expf(m[g] - mn);
          const float pg = expf(score - mn);
          l[g] = l[g] * corr + pg;
#pragma unroll
          for (int d = 0; d < DPL; ++d) acc[g][d] = fmaf(pg, vf[d], acc[g][d] * corr);
          m[g] = mn;
        }
      }
    }
    seq += (unsigned)it.nb;
    total += it.nb;
    trace_mark(trow, 6);
    // ---- the warps' states meet in shared memory: sh[(warp * GI + g) * rec ...]
#pragma unroll
    for (int g = 0; g < GI; ++g) {
      float* dst = sh + (size_t)(warp * GI + g) * rec;
#pragma unroll
      for (int d = 0; d < DPL; ++d) dst[lane * DPL + d] = acc[g][d];
      if (lane == 0) {
        dst[Dh] = m[g];
        dst[Dh + 1] = l[g];
      }
    }
    cons_sync();
    trace_mark(trow, 7);
    if (warp < GI) {
      // warp g merges the 7 states of head g in warp order and publishes the part record
      const int g = warp;
      float M = -INFINITY;
#pragma unroll 1
      for (int w2 = 0; w2 < kNWC; ++w2) M = fmaxf(M, sh[(size_t)(w2 * GI + g) * rec + Dh]);
      float L = 0.f, o[DPL];
#pragma unroll
      for (int d = 0; d < DPL; ++d) o[d] = 0.f;
#pragma unroll 1
      for (int w2 = 0; w2 < kNWC; ++w2) {
        const float* src = sh + (size_t)(w2 * GI + g) * rec;
        const float lw = src[Dh + 1];
        const float wgt = lw > 0.f ? expf(src[Dh] - M) : 0.f;
        L += lw * wgt;
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[d] = fmaf(src[lane * DPL + d], wgt, o[d]);
      }
      const int h = it.hg * GI + g;
      const size_t pi = ((size_t)it.b * H + h) * ap.cph + it.part;
#pragma unroll
      for (int d = 0; d < DPL; d += 2) st_tword2(st.part_acc, pi * Dh + lane * DPL + d, o[d], o[d + 1], tag_out);
      if (lane == 0) st_tword2(st.part_ml, pi * 2, M, L, tag_out);
    }
    trace_mark(trow, 8);
    cons_sync();   // the states in shared memory may be overwritten
  }
  return total;
}

template <typename T>
__device__ __forceinline__ int run_attn(const Stage& st, const CtaConst& cc, int s, unsigned seq_base) {
  const int G = qdiv(st.H, st.Hk);
  const int dpl = st.Dh / 32;
  if ((G & 1) == 0) {
    if (dpl == 4) return attn_stage<T, 2, 4>(st, cc, s, seq_base);
    return attn_stage<T, 2, 2>(st, cc, s, seq_base);
  }
  if (dpl == 4) return attn_stage<T, 1, 4>(st, cc, s, seq_base);
  return attn_stage<T, 1, 2>(st, cc, s, seq_base);
}

// Merges the part records into a plain [B, H*Dh] array of type T (or fp32): the last stage of a
// call whose result is the attention output itself.
template <typename T>
__device__ FSVD_COLD void run_attn_out(const Stage& st, const CtaConst& cc, int s, int gtid, int gthreads) {
  const Waiter w = {&cc, s};
  const int HD2 = (st.H * st.Dh) >> 1, units = st.B * HD2;
  const uint32_t tag = stage_tag(cc.tag_base, st.in_stage);
  for (int u = gtid; u < units; u += gthreads) {
    const int b = qdiv(u, HD2), e = (u - b * HD2) * 2;
    const int h = qdiv(e, st.Dh);
    const float2 o = attn_merge2(st, b, h, e - h * st.Dh, tag, w);
    const size_t i = (size_t)b * st.H * st.Dh + e;
    if (st.flags & SF_OUT_T) {
      TT<T>::st(st.out, i, o.x);
      TT<T>::st(st.out, i + 1, o.y);
    } else {
      reinterpret_cast<float*>(st.out)[i] = TT<T>::rnd(o.x);
      reinterpret_cast<float*>(st.out)[i + 1] = TT<T>::rnd(o.y);
    }
  }
}

// ----------------------------------------------------------------------------- small stages
template <typename T>
__device__ __forceinline__ void run_embed(const Stage& st, int gtid, int gthreads, uint32_t tag) {
  using X = TT<T>;
  const int d = st.P, B = st.B;
  for (int i = gtid; i < B * d; i += gthreads) {
    const int b = i / d, k = i - b * d;
    int tok = st.tokens[b];
    tok = min(max(tok, 0), st.vocab - 1);
    out_store<T>(st, st.out, (size_t)i, X::ld(st.WA, (size_t)tok * d + k), tag);
  }
}

// CTA 0 only.  Lowest index wins among equal maxima.
static __device__ FSVD_COLD void run_argmax(const Stage& st, float* redv, int* redi, int tid,
                                           int nthreads) {
  const int V = st.vocab, B = st.B;
  const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
  const float* logits = reinterpret_cast<const float*>(st.vl_src);
  int step = *st.step_counter;
  for (int b = 0; b < B; ++b) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int v0 = tid; v0 < V; v0 += nthreads * 8) {
      float x[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int v = v0 + q * nthreads;
        x[q] = v < V ? __ldcg(logits + (size_t)b * V + v) : -INFINITY;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int v = v0 + q * nthreads;
        if (v < V && (x[q] > best || (x[q] == best && v < bi))) {
          best = x[q];
          bi = v;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (lane == 0) {
      redv[warp] = best;
      redi[warp] = bi;
    }
    cons_sync();
    if (tid == 0) {
      for (int i = 1; i < nwarps; ++i)
        if (redv[i] > best || (redv[i] == best && redi[i] < bi)) {
          best = redv[i];
          bi = redi[i];
        }
      if (bi == 0x7fffffff) bi = 0;
      st.tokens[b] = bi;
      if (st.token_log && step < st.max_steps) st.token_log[(size_t)step * B + b] = bi;
      if (st.seqlens_rw) st.seqlens_rw[b] += 1;
    }
    cons_sync();
  }
  if (tid == 0) *st.step_counter = step + 1;
}

// ----------------------------------------------------------------------------- the kernel
// Dynamic shared memory layout:
//   [0, 2*sizeof(Stage))        current and next stage descriptor
//   [.., +2048)                 reduction scratch (256), flags and cache positions (256), CtaConst (512),
//                               column table of the running GEMV stage (1024)
//   [.., +kSmallProgBytes)      copy of a by-value program (per-op launches)
//   [.., +512)                  ring mbarriers: full[kMaxSlots], empty[kMaxSlots]
//   -- header rounded to 1 KB --
//   [.., +nslots*slot_bytes)    the ring (kBoxBytes slots; 8704 when the program streams int4 tiles)
//   [.., +part_bytes)           partial sums of the warps / attention scratch (sized by the host)
//   [.., +vec_bytes)            staged input vector, B rows of xstride elements
// Stage timeline (optional): trace[(s*grid + cta)*16 + k] = globaltimer at: 0 stage entry,
// 1 grid barrier passed, 2 vector staged, 3 stage done, 4 vector words arrived, 5 norm reduced,
// 7 boxes consumed, 8 plans made, 10 CTA synchronised, 11 epilogue done (attention: 4 query
// arrived, 5 boxes folded, 6 new rows folded, 7 states met, 8 part record stored).
template <typename T, bool Q4>
__global__ void __launch_bounds__(kThreads, 1)
fsvd_decode_kernel(const Stage* __restrict__ prog_global, const __grid_constant__ SmallProgram small,
                   const unsigned char* __restrict__ maps_global, const __grid_constant__ SmallMaps small_maps,
                   int use_small, int nstages, SyncState* sync, int xstride, int part_bytes,
                   int vec_bytes, int nslots, int slot_bytes, unsigned long long* trace, long long wait_limit,
                   int tune) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  unsigned char* cur_base = smem;
  float* red = reinterpret_cast<float*>(smem + 2 * kStageBytesAl);
  int* flags_sh = reinterpret_cast<int*>(smem + 2 * kStageBytesAl + 256);
  CtaConst* ccp = reinterpret_cast<CtaConst*>(smem + 2 * kStageBytesAl + 512);
  static_assert(sizeof(CtaConst) <= 512, "CtaConst must fit its shared-memory slot");
  Stage* small_sh = reinterpret_cast<Stage*>(smem + 2 * kStageBytesAl + kHeaderScratchBytes);
  unsigned char* bars = smem + 2 * kStageBytesAl + kHeaderScratchBytes + kSmallProgBytes;
  unsigned char* ring = smem + smem_header_bytes();
  float* part = reinterpret_cast<float*>(ring + (size_t)nslots * (Q4 ? slot_bytes : kBoxBytes));
  char* xvec = reinterpret_cast<char*>(part) + part_bytes;

  // Boxes past the K range hold zeros and multiply whatever follows the input in the staged
  // vector, so that memory must hold finite numbers from the start.
  for (int i = tid; i < vec_bytes / 16; i += kThreads)
    reinterpret_cast<uint4*>(xvec)[i] = make_uint4(0, 0, 0, 0);

  const Stage* prog = prog_global;
  const unsigned char* maps = maps_global;
  if (use_small) {
    // by-value program: copy it to shared memory once and walk it there; the TMA descriptors
    // stay in the parameter space
    const int* src = reinterpret_cast<const int*>(small.st);
    int* dst = reinterpret_cast<int*>(small_sh);
    const int nwords = nstages * (int)(sizeof(Stage) / 4);
    for (int i = tid; i < nwords; i += kThreads) dst[i] = src[i];
    prog = small_sh;
    maps = &small_maps.m[0][0];
  }
  // flags_sh[16..23]: positions of the batch rows
  if (tid < 8) {
    // read the descriptors where they came from: the shared-memory copy is still being written
    const Stage* src = use_small ? small.st : prog_global;
    const int* sl = nullptr;
    for (int s = 0; s < nstages && !sl; ++s) sl = src[s].seqlens;
    int B0 = 0;
    if (sl) B0 = src[0].B;
    flags_sh[16 + tid] = (sl && tid < B0) ? sl[tid] : 0;
    if (tid == 0) ccp->pc.ptr = sl;
  }
  if (tid == 0) {
    flags_sh[1] = 0;   // set when a wait ran out: nobody in this CTA waits again
    CtaConst& c = *ccp;
    c.ring.full = smem_u32(bars);
    c.ring.empty = c.ring.full + kMaxSlots * 8;
    c.ring.data = smem_u32(ring);
    c.ring.stride = Q4 ? (uint32_t)slot_bytes : (uint32_t)kBoxBytes;
    c.ring.ns = nslots;
    c.pc.pos = flags_sh + 16;
    c.sync = sync;
    c.giveup = reinterpret_cast<volatile int*>(flags_sh + 1);
    c.limit = wait_limit;
    c.tag_base = __ldcg(&sync->tag_base);
    c.trace = trace;
    c.xvec = xvec;
    c.red = red;
    c.part = part;
    c.xtab = reinterpret_cast<int*>(smem + 2 * kStageBytesAl + 1024);
    c.xstride = xstride;
    c.backoff_ns = ((tune >> 4) & 15) * 32;
    c.gate = (tune >> 8) & 1;
    c.cap = tune & 15;
    for (int i = 0; i < nslots; ++i) {
      mbar_init(c.ring.full + i * 8, 1);
      mbar_init(c.ring.empty + i * 8, 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  constexpr int kStageWords = (int)(sizeof(Stage) / 4);
  __syncthreads();
  if (tid < kStageWords)
    reinterpret_cast<int*>(cur_base)[tid] = reinterpret_cast<const int*>(prog)[tid];

  const CtaConst& cc = *ccp;
  if (warp >= kNWC) {
    // ---------------- producers
    producer_loop<T, Q4>(prog, nstages, maps, cc, lane);
  } else {
    // ---------------- consumers
    unsigned seq_base = 0, nbar = 0;
    for (int s = 0; s < nstages; ++s) {
      cons_sync();  // everybody is done with the previous stage's buffers; descriptor s landed
      const Stage& st = *reinterpret_cast<const Stage*>(cur_base + (s & 1) * kStageBytesAl);
      unsigned long long* trow = trace_row(cc, s);
      trace_mark(trow, 0);
      // the last consumer warp fetches the next descriptor while the others go on
      if (warp == kNWC - 1 && s + 1 < nstages) {
        int* dst = reinterpret_cast<int*>(cur_base + ((s + 1) & 1) * kStageBytesAl);
        const int* src = reinterpret_cast<const int*>(prog + s + 1);
        for (int i = lane; i < kStageWords; i += 32) dst[i] = src[i];
        __syncwarp();
        // What the next stage reads from HBM besides its boxes (norm weights, the rotary table rows
        // of the batch rows' positions) is asked for now: a cold read on the critical path costs
        // microseconds while the box stream saturates the memory system.
        const Stage& nx = *reinterpret_cast<const Stage*>(dst);
        if (nx.type == ST_GEMV) {
          if (nx.vl_mode == VL_RMSNORM) prefetch_l2(nx.vl_w, nx.vl_len * (int)sizeof(T), lane);
          if (nx.cos_tab && lane < nx.B) {
            const int half = nx.Dh >> 1;
            const size_t off = (size_t)min(cached_pos(cc.pc, nx.seqlens, lane), nx.S_max - 1) * half * sizeof(T);
            prefetch_l2(reinterpret_cast<const char*>(nx.cos_tab) + off, half * (int)sizeof(T), 0);
            prefetch_l2(reinterpret_cast<const char*>(nx.sin_tab) + off, half * (int)sizeof(T), 0);
          }
        }
      }
      const unsigned long long bar_target = (unsigned long long)(nbar + 1u) * gridDim.x;
      if (st.flags & SF_BARRIER) ++nbar;
      if (st.type == ST_GEMV) {
        seq_base += (unsigned)gemv_stage<T, Q4>(st, cc, s, seq_base, bar_target);
      } else {
        const Waiter w = {&cc, s};
        if (st.flags & SF_BARRIER) barrier_wait(w, bar_target, tid);
        trace_mark(trow, 1);
        if (st.type == ST_ATTN) {
          seq_base += (unsigned)run_attn<T>(st, cc, s, seq_base);
        } else if (st.type == ST_ATTN_OUT) {
          run_attn_out<T>(st, cc, s, blockIdx.x * kConsThreads + tid, gridDim.x * kConsThreads);
        } else if (st.type == ST_EMBED) {
          run_embed<T>(st, blockIdx.x * kConsThreads + tid, gridDim.x * kConsThreads, stage_tag(cc.tag_base, s));
        } else if (st.type == ST_ARGMAX) {
          if (blockIdx.x == 0) run_argmax(st, red, flags_sh + 8, tid, kConsThreads);
        }
      }
      if (st.flags & SF_ARRIVE) {
        // Grid-barrier arrival: one fence and one add per CTA.
        cons_sync();
        if (tid == 0) {
          // the CTA barrier orders every thread's stores before this fence (cumulativity)
          asm volatile("fence.acq_rel.gpu;" ::: "memory");
          asm volatile("red.relaxed.gpu.global.add.u64 [%0], 1;" ::"l"(&sync->arrivals) : "memory");
        }
      }
      trace_mark(trow, 3);
    }
  }
  __syncthreads();
  // After a give-up, copies may still be in flight towards this CTA's shared memory: give them
  // time to land before the CTA retires (bounded).
  if (flags_sh[1])
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  // The last CTA to finish leaves the words ready for the next launch: every CTA has passed all
  // its barriers and read tag_base before it can get here.
  if (tid == 0) {
    __threadfence();
    const unsigned long long tag_base = cc.tag_base;
    const unsigned done = atomicAdd(&sync->done_ctas, 1u);
    if (done == gridDim.x - 1) {
      sync->done_ctas = 0;
      sync->arrivals = 0;
      sync->tag_base = tag_base + (unsigned long long)nstages;
    }
  }
}

}  // namespace fsvd
