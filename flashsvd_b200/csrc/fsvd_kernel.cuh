// Persistent stage interpreter for single-token decode of low-rank (W = U·V) transformers.
//
// Launch geometry: one CTA per SM (cooperative launch), 7 consumer warps + 1 producer warp
// (7 issuing lanes).
//
// Factor stream.  A GEMV stage is cut into units of 16 factor rows x one K segment; units go
// round-robin to the CTAs.  A unit is a row of boxes, one box = 16 rows x 448 bytes (7 KB), and
// the boxes of all GEMV stages of the program, in program order, form the CTA's box sequence.
// The producer warp walks that sequence on its own: box number q goes into ring slot q % NS
// with one cp.async.bulk.tensor (TMA) as soon as the slot's previous content has been released.
// The factors do not depend on the activations, so the producers run ahead of the consumers by
// the whole ring (21 slots, 147 KB per SM), across stage boundaries and grid barriers: HBM keeps
// streaming while the CTAs synchronise.  Slot s is always consumed by warp s % 7 (NS is a
// multiple of 7) and filled by producer lane s % 7, so every mbarrier sees its phases in
// order from a single waiting thread or warp.
// (Measured on B200: this ring with real lds + mma consumers streams 6.4-6.9 TB/s; a single
// issuing thread tops out near 3.4 TB/s, two reach the HBM limit.)
//
// Arithmetic.  bf16: a box is the A operand (16 rows) of mma.sync.m16n8k16, the staged
// activation vector the B operand with the batch as N.  A dot product does not care about the
// order of k, so lane (g, t) feeds the k-slots it owns with 8 consecutive columns: one 16-byte
// shared-memory load of factor row g, one of row g + 8 and one of activation row g.  fp32
// (parity mode): the same loads, plain FMAs and a quad reduction by shuffles.  A warp adds its
// boxes of one (unit, operand) in registers and leaves the sum in shared memory; the sums of the
// warps are added in a fixed order and the stage's epilogue (RoPE + cache append, SiLU·up,
// residual, ...) runs on the result, so results do not depend on timing.
//
// All waits are bounded: a wait that runs out records an error code in SyncState::status and
// the kernel carries on without waiting again, so a fault in the protocol ends in an error
// return on the host, never in a hung device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <type_traits>
#include <utility>

#include "fsvd_stage.h"

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
template <int OFF>
__device__ __forceinline__ uint4 lds128_imm(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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
  static __device__ __forceinline__ float ldcg(const void* p, size_t i) {
    const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p) + i);
    return __uint_as_float((unsigned)u << 16);
  }
  static __device__ __forceinline__ void st(void* p, size_t i, float v) {
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
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
  static __device__ __forceinline__ float ldcg(const void* p, size_t i) {
    return __ldcg(reinterpret_cast<const float*>(p) + i);
  }
  static __device__ __forceinline__ void st(void* p, size_t i, float v) {
    reinterpret_cast<float*>(p)[i] = v;
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

// ----------------------------------------------------------------------------- GEMV stage
// Operands of an item's epilogue that do not depend on the accumulators; fetched when the item
// starts so that their latency hides behind the item's tiles.
// The operands stay as raw bits until the epilogue: converting a loaded bf16 to float right
// away would stall the warp on the load it was meant to hide.
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
// Cache positions seqlens[b] of the program's sequence-length array, read once per launch into
// shared memory (the array only changes in the last stage of a step).
struct PosCache {
  const int* ptr;   // the array the cached values come from
  const int* pos;   // shared memory, one entry per batch row
};
__device__ __forceinline__ int cached_pos(const PosCache& pc, const int* seqlens, int b) {
  return seqlens == pc.ptr ? pc.pos[b] : seqlens[b];
}

template <typename T>
__device__ __forceinline__ void epi_prefetch(const Stage& st, int p, int b, EpiAux& ax, const PosCache pc) {
  using X = TT<T>;
  ax.r0 = ax.r1 = 0u;
  ax.pos = 0;
  switch (st.epi) {
    case EPI_RESID: {
      const size_t i = (size_t)b * st.P + p;
      if (st.flags & SF_RESID_T) ax.r0 = raw_ld<T>(st.resid, i);
      else ax.r0 = raw_ld<float>(st.resid, i);
    } break;
    case EPI_ROPE_Q:
    case EPI_ROPE_K: {
      const int half = st.rope_half;
      const int j = qmod(p, half);
      ax.pos = cached_pos(pc, st.seqlens, b);
      const int pt = min(ax.pos, st.S_max - 1);   // a position past the tables is reported, not read
      ax.r0 = raw_ld<T>(st.cos_tab, (size_t)pt * half + j);
      ax.r1 = raw_ld<T>(st.sin_tab, (size_t)pt * half + j);
    } break;
    case EPI_V:
      ax.pos = cached_pos(pc, st.seqlens, b);
      break;
    case EPI_QKV: {
      const int half = st.rope_half;
      ax.pos = cached_pos(pc, st.seqlens, b);
      if (p < (st.H + st.Hk) * half) {   // q and k rows rotate
        const int j = qmod(p, half);
        const int pt = min(ax.pos, st.S_max - 1);
        ax.r0 = raw_ld<T>(st.cos_tab, (size_t)pt * half + j);
        ax.r1 = raw_ld<T>(st.sin_tab, (size_t)pt * half + j);
      }
    } break;
    default:
      break;
  }
}

template <typename T>
__device__ __forceinline__ void gemv_epilogue(const Stage& st, int p, int b, int seg, float a,
                                              float bsum, const EpiAux& ax) {
  using X = TT<T>;
  const int P = st.P;
  switch (st.epi) {
    case EPI_PARTIAL: {
      const size_t i = ((size_t)seg * st.B + b) * P + p;
      reinterpret_cast<float*>(st.out)[i] = a;
    } break;
    case EPI_STORE: {
      const float v = X::rnd(a);
      const size_t i = (size_t)b * P + p;
      if (st.flags & SF_OUT_T) X::st(st.out, i, v);
      else reinterpret_cast<float*>(st.out)[i] = v;
    } break;
    case EPI_RESID: {
      const size_t i = (size_t)b * P + p;
      const float res = (st.flags & SF_RESID_T) ? raw_to_float<T>(ax.r0) : __uint_as_float(ax.r0);
      const float v = X::rnd(res + X::rnd(a));
      if (st.flags & SF_OUT_T) X::st(st.out, i, v);
      else reinterpret_cast<float*>(st.out)[i] = v;
    } break;
    case EPI_SWIGLU: {
      const float g = X::rnd(a), u = X::rnd(bsum);
      const float sg = X::rnd(g / (1.0f + expf(-g)));
      const float v = X::rnd(sg * u);
      const size_t i = (size_t)b * P + p;
      if (st.flags & SF_OUT_T) X::st(st.out, i, v);
      else reinterpret_cast<float*>(st.out)[i] = v;
    } break;
    case EPI_ROPE_Q:
    case EPI_ROPE_K: {
      const int half = st.rope_half;
      const int h = qdiv(p, half), j = p - h * half;
      const int pos = ax.pos;
      const float c = raw_to_float<T>(ax.r0), sn = raw_to_float<T>(ax.r1);
      const float x1 = X::rnd(a), x2 = X::rnd(bsum);
      const float o1 = X::rnd(X::rnd(x1 * c) - X::rnd(x2 * sn));
      const float o2 = X::rnd(X::rnd(x2 * c) + X::rnd(x1 * sn));
      if (st.epi == EPI_ROPE_Q) {
        const size_t base = ((size_t)b * st.H + h) * st.Dh + j;
        if (st.flags & SF_OUT_T) {
          X::st(st.out, base, o1);
          X::st(st.out, base + half, o2);
        } else {
          float* q = reinterpret_cast<float*>(st.out);
          q[base] = o1;
          q[base + half] = o2;
        }
      } else if (pos < st.S_max) {
        const size_t base = (((size_t)cache_row(st, b) * st.S_max + pos) * st.Hk + h) * st.Dh + j;
        X::st(st.cache, base, o1);
        X::st(st.cache, base + half, o2);
      }
    } break;
    case EPI_V: {
      const int pos = ax.pos;
      if (pos < st.S_max)
        X::st(st.cache, ((size_t)cache_row(st, b) * st.S_max + pos) * ((size_t)st.Hk * st.Dh) + p, X::rnd(a));
    } break;
    case EPI_QKV: {
      const int half = st.rope_half, pos = ax.pos;
      const int hh = qdiv(p, half), j = p - hh * half;   // head over [q heads | k heads | v heads]
      const float x1 = X::rnd(a), x2 = X::rnd(bsum);
      if (hh < st.H + st.Hk) {
        const float c = raw_to_float<T>(ax.r0), sn = raw_to_float<T>(ax.r1);
        const float o1 = X::rnd(X::rnd(x1 * c) - X::rnd(x2 * sn));
        const float o2 = X::rnd(X::rnd(x2 * c) + X::rnd(x1 * sn));
        if (hh < st.H) {
          const size_t base = ((size_t)b * st.H + hh) * st.Dh + j;
          if (st.flags & SF_OUT_T) {
            X::st(st.out, base, o1);
            X::st(st.out, base + half, o2);
          } else {
            float* q = reinterpret_cast<float*>(st.out);
            q[base] = o1;
            q[base + half] = o2;
          }
        } else if (pos < st.S_max) {
          const size_t base = (((size_t)cache_row(st, b) * st.S_max + pos) * st.Hk + (hh - st.H)) * st.Dh + j;
          X::st(st.cache, base, o1);
          X::st(st.cache, base + half, o2);
        }
      } else if (pos < st.S_max) {
        void* vc = const_cast<void*>(st.vcache);
        const size_t base = (((size_t)cache_row(st, b) * st.S_max + pos) * st.Hk + (hh - st.H - st.Hk)) * st.Dh + j;
        X::st(vc, base, x1);
        X::st(vc, base + half, x2);
      }
    } break;
    default:
      break;
  }
}

// ----------------------------------------------------------------------------- global loads
// Activations, partial sums and cache rows are produced by other CTAs of the same launch; they
// are read with ld.global.cg (L2 only) so that no stale line of this SM's L1 can be returned.
__device__ __forceinline__ float4 ldcg_f4(const void* p) {
  return __ldcg(reinterpret_cast<const float4*>(p));
}
// 4 consecutive elements at element index i (i % 4 == 0) of an fp32 or T array, as fp32.
template <typename T>
__device__ __forceinline__ float4 ld4(const void* base, size_t i, bool is_T);
template <>
__device__ __forceinline__ float4 ld4<float>(const void* base, size_t i, bool) {
  return ldcg_f4(reinterpret_cast<const float*>(base) + i);
}
template <>
__device__ __forceinline__ float4 ld4<__nv_bfloat16>(const void* base, size_t i, bool is_T) {
  if (!is_T) return ldcg_f4(reinterpret_cast<const float*>(base) + i);
  const uint2 u = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + i));
  return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                     __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
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

// DPL consecutive elements of a T array (cache row, L2 only), as fp32.
template <typename T, int DPL>
__device__ __forceinline__ void ld_row(const void* base, size_t i, float* out);
template <>
__device__ __forceinline__ void ld_row<__nv_bfloat16, 4>(const void* base, size_t i, float* o) {
  const uint2 u = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + i));
  o[0] = __uint_as_float(u.x << 16); o[1] = __uint_as_float(u.x & 0xffff0000u);
  o[2] = __uint_as_float(u.y << 16); o[3] = __uint_as_float(u.y & 0xffff0000u);
}
template <>
__device__ __forceinline__ void ld_row<__nv_bfloat16, 2>(const void* base, size_t i, float* o) {
  const uint32_t u = __ldcg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(base) + i));
  o[0] = __uint_as_float(u << 16); o[1] = __uint_as_float(u & 0xffff0000u);
}
template <>
__device__ __forceinline__ void ld_row<float, 4>(const void* base, size_t i, float* o) {
  const float4 v = ldcg_f4(reinterpret_cast<const float*>(base) + i);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <>
__device__ __forceinline__ void ld_row<float, 2>(const void* base, size_t i, float* o) {
  const float2 v = __ldcg(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(base) + i));
  o[0] = v.x; o[1] = v.y;
}
// ----------------------------------------------------------------------------- vector stage-in
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

// Brings the stage's input vector into shared memory as T.  All global loads of a thread are
// issued before the first use so that their L2 latencies overlap.  Sources of type T are copied
// or normalised in 16-byte units; fp32 partial sums are added in segment order, then rounded.
template <typename T>
__device__ __forceinline__ void stage_vector(const Stage& st, char* xvec, int xstride, float* red,
                                          int tid, int nthreads, unsigned long long* trow) {
  using X = TT<T>;
  constexpr int VEC = X::kVec;  // elements per 16 bytes of T
  const int len = st.vl_len, B = st.B;
  const bool inT = (st.flags & SF_IN_T) != 0;
  if (st.vl_mode == VL_SUM && inT) {
    // T -> T copy (nseg is 1 for every T source); with SF_SEG_X only the K segment of this CTA
    // (no unrolling: with segments staged per CTA a thread copies one or two 16-byte pieces, and
    // the interpreter's code has to stay small - its cold paths are bound by instruction fetch)
    constexpr int U = 1;
    int col0 = 0, lenS = len;
    if (st.flags & SF_SEG_X) {
      const int grid = gridDim.x;
      const int seg = qmod(first_item(blockIdx.x, qmod(st.rot, grid), grid), st.segs);
      const int kseg = (st.flags & SF_Q4) ? st.cps * kQ4BoxCols : st.cps * (kBoxRowBytes / (int)sizeof(T));
      col0 = seg * kseg;
      lenS = len - col0 < kseg ? len - col0 : kseg;
      if (lenS < 0) lenS = 0;
    }
    const int upr = lenS / VEC, units = B * upr;
    for (int u0 = tid; u0 < units; u0 += nthreads * U) {
      uint4 v[U];
#pragma unroll
      for (int q = 0; q < U; ++q) {
        const int u = u0 + q * nthreads;
        if (u < units) {
          const int b = qdiv(u, upr), k = (u - b * upr) * VEC;
          v[q] = ld_raw16<T>(st.vl_src, (size_t)b * len + col0 + k);
        }
      }
#pragma unroll
      for (int q = 0; q < U; ++q) {
        const int u = u0 + q * nthreads;
        if (u < units) {
          const int b = qdiv(u, upr), k = (u - b * upr) * VEC;
          *reinterpret_cast<uint4*>(xvec + ((size_t)b * xstride + k) * sizeof(T)) = v[q];
        }
      }
    }
  } else if (st.vl_mode == VL_SUM) {
    // fp32 partial sums [nseg][B][len]; with few segments a thread handles up to UP float4
    // positions per pass and issues all their loads before the first add (one memory round trip
    // per pass instead of one per position)
    constexpr int SMAX = 8;  // kMaxSegs of the program builder
    constexpr int UP = 4;
    const int nseg = st.vl_nseg;
    const int upr = len >> 2, units = B * upr;
    const size_t segstride = (size_t)B * len;
    const float* src = reinterpret_cast<const float*>(st.vl_src);
    if (nseg <= 3) {
      for (int u0 = tid; u0 < units; u0 += nthreads * UP) {
        float4 v[UP][3];
#pragma unroll
        for (int k = 0; k < UP; ++k) {
          const int u = u0 + k * nthreads;
#pragma unroll
          for (int q = 0; q < 3; ++q)
            if (q < nseg && u < units) v[k][q] = ldcg_f4(src + q * segstride + (size_t)u * 4);
        }
#pragma unroll
        for (int k = 0; k < UP; ++k) {
          const int u = u0 + k * nthreads;
          if (u < units) {
            float4 a = v[k][0];
#pragma unroll
            for (int q = 1; q < 3; ++q)
              if (q < nseg) { a.x += v[k][q].x; a.y += v[k][q].y; a.z += v[k][q].z; a.w += v[k][q].w; }
            const int b = qdiv(u, upr), k2 = (u - b * upr) * 4;
            st4<T>(xvec, (size_t)b * xstride + k2, a);
          }
        }
      }
    } else {
      for (int u = tid; u < units; u += nthreads) {
        float4 v[SMAX];
#pragma unroll
        for (int q = 0; q < SMAX; ++q)
          if (q < nseg) v[q] = ldcg_f4(src + q * segstride + (size_t)u * 4);
        float4 a = v[0];
#pragma unroll
        for (int q = 1; q < SMAX; ++q)
          if (q < nseg) { a.x += v[q].x; a.y += v[q].y; a.z += v[q].z; a.w += v[q].w; }
        const int b = qdiv(u, upr), k = (u - b * upr) * 4;
        st4<T>(xvec, (size_t)b * xstride + k, a);
      }
    }
  } else if (st.vl_mode == VL_RMSNORM) {
    // T source, weight of type T; a row longer than the register window is read twice
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

// ----------------------------------------------------------------------------- waits
// The budget of a bounded wait, in SM clocks: 8 bytes of shared memory behind the CTA's give-up flag
// (the flag is set by the first wait of the CTA that runs out: nobody in the CTA waits again).
__device__ __forceinline__ long long wait_budget(volatile int* giveup) {
  return *reinterpret_cast<volatile long long*>(giveup + 1);
}
// Grid barrier wait (one polling lane per CTA) in front of a stage with SF_BARRIER.
__device__ __forceinline__ void barrier_wait(SyncState* sync, volatile int* giveup, unsigned long long target, int s,
                                             int tid) {
  if (tid == 0) {
    if (ld_acquire_u64(&sync->arrivals) < target) {
      const long long c0 = clock64();
      unsigned spins = 0;
      while (ld_acquire_u64(&sync->arrivals) < target) {
        if ((++spins & 63u) == 0) {
          if (*giveup) break;
          if (clock64() - c0 > wait_budget(giveup)) {
            if (atomicCAS(&sync->status, (int)DS_OK, (int)DS_BARRIER_TIMEOUT) == (int)DS_OK) sync->status_detail = s;
            *giveup = 1;
            break;
          }
        }
      }
    }
  }
  cons_sync();
}

// Bounded wait on a ring mbarrier.  False: the wait ran out (recorded in SyncState::status) or
// this CTA has already given up; the caller goes on without the data.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, SyncState* sync,
                                          volatile int* giveup, int detail) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*giveup) return false;
  const long long c0 = clock64();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 127u) == 0) {
      if (*giveup) return false;
      if (clock64() - c0 > wait_budget(giveup)) {
        if (atomicCAS(&sync->status, (int)DS_OK, (int)DS_COPY_TIMEOUT) == (int)DS_OK) sync->status_detail = detail;
        *giveup = 1;
        return false;
      }
    }
  }
  return true;
}

// ----------------------------------------------------------------------------- GEMV engine
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

struct Ring {
  uint32_t full, empty;   // shared-memory addresses of the mbarrier arrays
  uint32_t data;          // shared-memory address of slot 0
  uint32_t stride;        // bytes between slots (kBoxBytes, or kQ4BoxBytes when the program has int4 stages)
  int ns;                 // slots, a multiple of kNWC (or fewer than kNWC)
};

// The producer warp.  Lane L < N (N = 7, or the slot count of a smaller ring) owns the boxes
// q with q % N == L, which always land in the slots s with s % N == L: a lane waits only on the
// mbarriers of its own slots and sees their phases in order (a parity wait cannot tell phase k
// from phase k + 2).  The lanes walk the CTA's box sequence of the whole program in lockstep, N
// boxes per round: every lane keeps its own cursor (stage, unit, operand, chunk), waits for its
// slot, and then all lanes issue their TMA copies with one instruction.  (Lanes that ran their
// own loops and met at different barriers serialised: 1 such lane gave 354, 4 lanes 327, 8 lanes
// 298 tokens/s on the 7B-shape model.)
template <typename T, bool Q4>
__device__ __forceinline__ void producer_loop(const Stage* prog, int nstages, const unsigned char* maps,
                                           const Ring rg, int lane, SyncState* sync, volatile int* giveup) {
  constexpr int BOXCOLS = kBoxRowBytes / (int)sizeof(T);
  const int grid = gridDim.x, cta = blockIdx.x;
  const int N = rg.ns < kNWC ? rg.ns : kNWC;
  const unsigned mask = (1u << N) - 1u;
  if (lane >= N) return;
  // cursor of this lane
  int s = -1, j = 0, op = 0, c = 0;          // stage, unit ordinal, operand, chunk
  int nu = 0, nops = 1, cps = 1, first = 0, segs = 1, half = 0;
  int nch = 0;                               // > 0: the stage streams int4 tiles, nch per tile row
  const unsigned char* mapA = maps;
  bool done = false;
  // moves the cursor to the first box of the next GEMV stage with boxes for this CTA
  auto next_stage = [&]() {
    for (++s; s < nstages; ++s) {
      const Stage& st = prog[s];
      if (st.type != ST_GEMV) continue;
      const BoxPlan bp = plan_boxes(st.P, st.segs, st.cps, st.rot, st.WB != nullptr, cta, grid);
      if (bp.nbox == 0) continue;
      nu = bp.nu; nops = bp.nops; cps = bp.cps; first = bp.first; segs = st.segs; half = st.rope_half;
      nch = (Q4 && (st.flags & SF_Q4)) ? st.nch : 0;
      mapA = maps + (size_t)(2 * s) * 128;
      j = op = c = 0;
      return;
    }
    done = true;
  };
  // advances the cursor by k boxes
  auto advance = [&](int k) {
    while (k > 0 && !done) {
      const int room = cps - c;
      if (k < room) {
        c += k;
        k = 0;
      } else {
        k -= room;
        c = 0;
        if (++op == nops) {
          op = 0;
          if (++j == nu) next_stage();
        }
      }
    }
  };
  next_stage();
  advance(lane);
  int slot = lane, round = 0;
  while (__any_sync(mask, !done)) {
    bool ok = !done;
    if (ok && round > 0) ok = mbar_wait(rg.empty + slot * 8, (uint32_t)(round - 1) & 1u, sync, giveup, s);
    __syncwarp(mask);
    if (ok) {
      const int uidx = first + j * grid;
      const int grp = qdiv(uidx, segs), seg = uidx - grp * segs;
      const uint32_t fb = rg.full + slot * 8;
      const uint32_t dst = rg.data + (uint32_t)slot * (Q4 ? rg.stride : (uint32_t)kBoxBytes);
      if (Q4 && nch > 0) {
        // tile (row group, chunk) of the int4 stream; a chunk past the last tile of the row (the
        // tail of the last K segment) is fetched from outside the tensor and arrives as zeros
        // (zero scales)
        const int chunk = seg * cps + c;
        const int trow = phys_row(half, grp * kUnitRows) / kUnitRows;
        const int y = chunk < nch ? (trow * nch + chunk) * kQ4TileRows : 0x40000000;
        mbar_expect_tx(fb, kQ4BoxBytes);
        tma_box_2d(dst, mapA + (op ? 128 : 0), 0, y, fb);
      } else {
        mbar_expect_tx(fb, kBoxBytes);
        tma_box_2d(dst, mapA + (op ? 128 : 0), (seg * cps + c) * BOXCOLS, phys_row(half, grp * kUnitRows), fb);
      }
    } else if (!done) {
      done = true;   // a wait ran out: this lane stops (the consumers give up on their own)
    }
    advance(N);
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

// Per-stage context handed to the stage functions.
struct StageCtx {
  int s;
  SyncState* sync;
  unsigned long long bar_target;   // arrival count that opens this stage's barrier
  char* xvec;
  int xstride;
  float* red;
  float* part;                     // partial sums: [unit ordinal * nops + operand][kk][batch][16 rows]
  Ring ring;
  unsigned seq_base;               // boxes of this CTA in the stages before this one
  volatile int* giveup;
  PosCache pc;
  unsigned long long* trow;
};

// One GEMV stage, consumer warps.  Returns the number of boxes of this CTA in the stage.
template <typename T, bool Q4>
__device__ __forceinline__ int gemv_stage(const Stage& st, const StageCtx cx) {
  using X = TT<T>;
  constexpr int BOXCOLS = kBoxRowBytes / (int)sizeof(T);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int B = st.B, grid = gridDim.x, segs = st.segs;
  const BoxPlan bp = plan_boxes(st.P, segs, st.cps, st.rot, st.WB != nullptr, blockIdx.x, grid);
  const int cps = bp.cps, nops = bp.nops;
  const int rowsB = kUnitRows * B;
  const bool q4 = Q4 && sizeof(T) == 2 && (st.flags & SF_Q4);
  const int boxcols = (Q4 && q4) ? kQ4BoxCols : BOXCOLS;

  // operands of the epilogues this thread will run (outputs tid and tid + 224), fetched now so
  // that their latency hides behind the barrier and the streaming
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
      if (p < st.P) epi_prefetch<T>(st, p, b, ax0, cx.pc);
    }
    if (tid + kConsThreads < nout) {
      out_pos(tid + kConsThreads, j, b, r, seg, p);
      if (p < st.P) epi_prefetch<T>(st, p, b, ax1, cx.pc);
    }
  }

  trace_mark(cx.trow, 8);
  // ---- wait for the producers of the input vector, stage it
  // A token at a position beyond the cache is not stored (the epilogues skip it) and is reported:
  // the reference's cache raises IndexError there (runtime/cache/attn_dense_kv.py:295-298).
  if ((st.epi == EPI_ROPE_K || st.epi == EPI_V || st.epi == EPI_QKV) && tid < st.B &&
      cached_pos(cx.pc, st.seqlens, tid) >= st.S_max)
    atomicCAS(&cx.sync->status, (int)DS_OK, (int)DS_CACHE_FULL);
  if (st.flags & SF_BARRIER) barrier_wait(cx.sync, cx.giveup, cx.bar_target, cx.s, tid);
  trace_mark(cx.trow, 1);
  if (st.vl_mode != VL_NONE) {
    stage_vector<T>(st, cx.xvec, cx.xstride, cx.red, tid, kConsThreads, cx.trow);
    cons_sync();
  }
  trace_mark(cx.trow, 2);

  // ---- this warp's boxes: local box l belongs to warp (seq_base + l) % step
  const int g = lane >> 2, t = lane & 3;
  const uint32_t xrow_bytes = (uint32_t)cx.xstride * (uint32_t)sizeof(T);
  const uint32_t xvec_s = smem_u32(cx.xvec) + t * 16;
  const uint32_t xlane_s = xvec_s + (uint32_t)(g < B ? g : 0) * xrow_bytes;
  const uint32_t wlane = (uint32_t)g * ((Q4 && q4) ? kQ4RowBytes : kBoxRowBytes) + t * 16;
  // Box number q is consumed by warp q % step: step = 7 for a ring of 7, 14 or 21 slots; a ring
  // of fewer than 7 slots (huge input vectors) has one warp per slot and leaves the others idle.
  const int step = cx.ring.ns < kNWC ? cx.ring.ns : kNWC;
  const int KK = cps < step ? cps : step;   // warps that hold partial sums of one (unit, operand)
  int l = warp < step ? qmod(warp - qmod((int)cx.seq_base, step) + step, step) : bp.nbox;
  int slot, round;
  {
    const unsigned seq0 = cx.seq_base + (unsigned)l;
    round = qdiv((int)seq0, cx.ring.ns);
    slot = (int)(seq0 - (unsigned)round * cx.ring.ns);
  }
  int io = qdiv(l, cps), c = l - io * cps;   // (unit ordinal * nops + operand), chunk inside it
  int cur_io = -1, cur_kk = 0, xcol0 = 0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};          // bf16: mma accumulators (rows g, g+8; batch 2t, 2t+1)
  float accf[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // fp32: [row half][batch]
  auto flush = [&]() {
    float* dst = cx.part + ((size_t)cur_io * KK + cur_kk) * rowsB;
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
      cur_kk = qmod(c, step);
      const int j = nops == 2 ? (io >> 1) : io, op = nops == 2 ? (io & 1) : 0;
      const int uidx = bp.first + j * grid;
      const int seg = qmod(uidx, segs);
      xcol0 = (op ? st.xB_off : st.xA_off) + ((st.flags & SF_SEG_X) ? 0 : seg * cps * boxcols);
      if (st.epi == EPI_QKV) {   // segs == 1: uidx is the row group; the part's input starts at part * K
        const int p0 = uidx * kUnitRows, half = st.rope_half;
        xcol0 += ((p0 >= st.H * half) + (p0 >= (st.H + st.Hk) * half)) * st.K;
      }
    }
    bool ok = mbar_wait(cx.ring.full + slot * 8, (uint32_t)round & 1u, cx.sync, cx.giveup, cx.s);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const uint32_t wb = cx.ring.data + (uint32_t)slot * (Q4 ? cx.ring.stride : (uint32_t)kBoxBytes) + wlane;
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
        for (int q = 0; q < 6; q += 2) {
          const uint4 xv = lds128(xb + q * 64), xw = lds128(xb + q * 64 + 64);
          const uint4 lo = lds128(wb + q * 64), lp = lds128(wb + q * 64 + 64);
          const uint4 hi = lds128(wb + 8 * kBoxRowBytes + q * 64), hj = lds128(wb + 8 * kBoxRowBytes + q * 64 + 64);
          mma_bf16_16816(a0, lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
          mma_bf16_16816(a1, lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
          mma_bf16_16816(a2, lp.x, hj.x, lp.y, hj.y, xw.x, xw.y);
          mma_bf16_16816(a3, lp.z, hj.z, lp.w, hj.w, xw.z, xw.w);
        }
        {
          constexpr int q = 6;
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
        for (int q = 0; q < 7; ++q) {
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
    if (lane == 0) mbar_arrive(cx.ring.empty + slot * 8);
    slot += step;
    if (slot >= cx.ring.ns) {
      slot -= cx.ring.ns;
      ++round;
    }
    c += step;
    while (c >= cps) {
      c -= cps;
      ++io;
    }
  }
  if (cur_io >= 0) flush();
  trace_mark(cx.trow, 7);
  cons_sync();
  trace_mark(cx.trow, 10);

  // ---- add the warps' partial sums in chunk order and run the epilogue
  for (int o = tid, it = 0; o < nout; o += kConsThreads, ++it) {
    int j, b, r, seg, p;
    out_pos(o, j, b, r, seg, p);
    if (p >= st.P) continue;
    EpiAux ax;
    if (it == 0) ax = ax0;
    else if (it == 1) ax = ax1;
    else epi_prefetch<T>(st, p, b, ax, cx.pc);
    const float* src = cx.part + ((size_t)(j * nops) * KK) * rowsB + b * 16 + r;
    float sum0 = 0.f, sum1 = 0.f;
    for (int k2 = 0; k2 < KK; ++k2) sum0 += src[(size_t)k2 * rowsB];
    if (nops == 2)
      for (int k2 = 0; k2 < KK; ++k2) sum1 += src[(size_t)(KK + k2) * rowsB];
    gemv_epilogue<T>(st, p, b, seg, sum0, sum1, ax);
  }
  trace_mark(cx.trow, 11);
  return bp.nbox;
}

// ----------------------------------------------------------------------------- attention stage
// Raw cache row piece of one lane: DPL consecutive elements of type T, kept packed in registers
// until they are used.
template <typename T, int DPL>
struct RawRow;
template <>
struct RawRow<__nv_bfloat16, 4> {
  uint2 v;
  __device__ __forceinline__ void load(const char* p, bool on) {
    v = make_uint2(0u, 0u);
    if (on) v = __ldcg(reinterpret_cast<const uint2*>(p));
  }
  __device__ __forceinline__ void unpack(float* o) const {
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
  }
};
template <>
struct RawRow<__nv_bfloat16, 2> {
  uint32_t v;
  __device__ __forceinline__ void load(const char* p, bool on) {
    v = 0u;
    if (on) v = __ldcg(reinterpret_cast<const uint32_t*>(p));
  }
  __device__ __forceinline__ void unpack(float* o) const {
    o[0] = __uint_as_float(v << 16); o[1] = __uint_as_float(v & 0xffff0000u);
  }
};
template <>
struct RawRow<float, 4> {
  float4 v;
  __device__ __forceinline__ void load(const char* p, bool on) {
    v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (on) v = __ldcg(reinterpret_cast<const float4*>(p));
  }
  __device__ __forceinline__ void unpack(float* o) const { o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
};
template <>
struct RawRow<float, 2> {
  float2 v;
  __device__ __forceinline__ void load(const char* p, bool on) {
    v = make_float2(0.f, 0.f);
    if (on) v = __ldcg(reinterpret_cast<const float2*>(p));
  }
  __device__ __forceinline__ void unpack(float* o) const { o[0] = v.x; o[1] = v.y; }
};

// Attention of the new token over the dense cache, CTA-cooperative.
//
// A head group = GI query heads that share one kv head (GI = 1, or 2 when H/Hk is even).  Its keys
// are cut into nsplit = cph * 7 splits: cph CTAs per head group, and in each of them the 7
// consumer warps take one split each.  Lane l owns dims [l*DPL, (l+1)*DPL) of the head.  The
// keys and values of a split are fetched in chunks of KMAX rows whose loads are all issued
// before the first use (one memory round trip per chunk; a split of the benchmark shape is one
// chunk); scores of a chunk are independent dot products and softmax runs once per chunk.
// The 7 partial results of a CTA meet in shared memory and are merged in warp order.  With
// cph == 1 that is the result; otherwise the CTA publishes its part and the last of the cph
// CTAs to arrive (atomic counter) merges the parts in part order, so the result does not depend
// on timing.
// What the attention stage needs to wait at its grid barrier itself: the item's index arithmetic
// (and the instruction fetch of this code) then happens while the CTA would be waiting anyway.
struct AttnBarrier {
  bool need;
  SyncState* sync;
  volatile int* giveup;
  unsigned long long target;
  int s;
};
template <typename T, int GI, int DPL>
__device__ __forceinline__ void attn_cta(const Stage& st, float* sh, const PosCache pc, const AttnBarrier ab) {
  using X = TT<T>;
  // Rows per chunk: a split of the benchmark shape (18 keys) takes two chunks of 10 rather than one
  // of 20 - half the unrolled code; the stage is bound by instruction fetch, not by the loads
  // (measured: 20 rows 407.7, 10 rows 411.5, 9 rows 405.8, 6 rows 401.7 tokens/s).
  constexpr int KBASE = (GI == 1) ? 10 : 12;
  constexpr int KMAX = sizeof(T) == 2 ? KBASE : KBASE / 2;   // rows in registers
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int Dh = st.Dh, H = st.H, B = st.B, grid = gridDim.x;
  const int R = qdiv(H, st.Hk) / GI;       // head groups per kv head
  const int Hg = st.Hk * R;                // head groups per batch row
  const int nsplit = st.nsplit, cph = nsplit / kNWC;
  const int nslice = B * Hg * cph;         // (batch row, head group, part)
  const size_t kv_row = (size_t)st.Hk * Dh;
  const bool qT = (st.flags & SF_IN_T) != 0;
  const int rec = Dh + 2;                  // floats of one partial result: acc[Dh], max, sum
  constexpr int ROWS = GI * KMAX;          // scores of one chunk
  static_assert(ROWS <= 32, "one score per lane");
  // per-warp scratch behind the partial results: score tile [ROWS][33] and probabilities [ROWS]
  float* const tile = sh + kNWC * GI * rec + warp * (ROWS * 34);
  float* const pbuf = tile + ROWS * 33;

  bool waited = !ab.need;
  for (int hs = first_item(blockIdx.x, qmod(st.rot, grid), grid); hs < nslice; hs += grid) {
    const int hq = qdiv(hs, cph), part = hs - hq * cph;
    const int b = qdiv(hq, Hg), hg = hq - b * Hg;
    const int hk = qdiv(hg, R);
    const int sp = part * kNWC + warp;
    const int n = min(cached_pos(pc, st.seqlens, b) + st.seqlen_add, st.S_max);
    const int per = qdiv(n + nsplit - 1, nsplit);
    const int j0 = sp * per, j1 = min(n, j0 + per);
    const size_t base = ((size_t)cache_row(st, b) * st.S_max) * kv_row + (size_t)hk * Dh + lane * DPL;
    const size_t row_bytes = kv_row * sizeof(T);
    const char* kbase = reinterpret_cast<const char*>(st.kcache) + base * sizeof(T);
    const char* vbase = reinterpret_cast<const char*>(st.vcache) + base * sizeof(T);

    // The key and the value rows of a chunk are requested together (one memory round trip per
    // chunk).  Rows are addressed by one running pointer and rows past the split are skipped by
    // predicate (their registers read as zeros).
    RawRow<T, DPL> kr[KMAX], vr[KMAX];
    auto fetch = [&](int c0) {
      const char* kp = kbase + (size_t)c0 * row_bytes;
      const char* vp = vbase + (size_t)c0 * row_bytes;
#pragma unroll
      for (int u = 0; u < KMAX; ++u) {
        kr[u].load(kp, c0 + u < j1);
        kp += row_bytes;
      }
#pragma unroll
      for (int u = 0; u < KMAX; ++u) {
        vr[u].load(vp, c0 + u < j1);
        vp += row_bytes;
      }
    };
    if (!waited) {
      barrier_wait(ab.sync, ab.giveup, ab.target, ab.s, tid);
      waited = true;
    }
    fetch(j0);
    float q[GI][DPL], acc[GI][DPL], m[GI], l[GI];
#pragma unroll
    for (int g = 0; g < GI; ++g) {
      const size_t qi = ((size_t)b * H + hg * GI + g) * Dh + lane * DPL;
      if (qT) {
        ld_row<T, DPL>(st.q, qi, q[g]);
      } else {
        ld_row<float, DPL>(st.q, qi, q[g]);
      }
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[g][d] = 0.f;
      m[g] = -INFINITY;
      l[g] = 0.f;
    }
    for (int c0 = j0; c0 < j1; c0 += KMAX) {
      if (c0 > j0) fetch(c0);
      // Partial dot products (this lane's dims) go to a [key][lane] tile in shared memory; lane r
      // then adds row r, so that every lane owns one full score: softmax costs one exp per lane
      // and 2 x 5 shuffles per head instead of 5 shuffles and one exp per key.
#pragma unroll
      for (int u = 0; u < KMAX; ++u) {
        float kf[DPL];
        kr[u].unpack(kf);
#pragma unroll
        for (int g = 0; g < GI; ++g) {
          float s2 = 0.f;
#pragma unroll
          for (int d = 0; d < DPL; ++d) s2 = fmaf(q[g][d], kf[d], s2);
          tile[(g * KMAX + u) * 33 + lane] = s2;
        }
      }
      __syncwarp();
      float sa = 0.f, sb = 0.f, sc2 = 0.f, sd = 0.f;
      if (lane < ROWS) {
        const float* row = tile + lane * 33;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          sa += row[i];
          sb += row[i + 1];
          sc2 += row[i + 2];
          sd += row[i + 3];
        }
      }
      const int gu = lane / KMAX, uu = lane - gu * KMAX;   // head and key of this lane's score
      const bool valid = lane < ROWS && c0 + uu < j1;
      const float score = valid ? ((sa + sb) + (sc2 + sd)) * st.scale : -INFINITY;
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
      if (lane < ROWS) pbuf[lane] = pmine;
      __syncwarp();
#pragma unroll
      for (int u = 0; u < KMAX; ++u) {
        float vf[DPL];
        vr[u].unpack(vf);
#pragma unroll
        for (int g = 0; g < GI; ++g) {
          const float pg = pbuf[g * KMAX + u];
#pragma unroll
          for (int d = 0; d < DPL; ++d) acc[g][d] = fmaf(pg, vf[d], acc[g][d]);
        }
      }
      __syncwarp();   // the tile is rewritten by the next chunk
    }
    // ---- the 7 partial results of the CTA meet in shared memory: sh[(warp * GI + g) * rec ...]
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
    if (warp < GI) {
      // warp g merges the 7 partial results of head g in warp order
      const int g = warp;
      float M = -INFINITY;
#pragma unroll
      for (int w2 = 0; w2 < kNWC; ++w2) M = fmaxf(M, sh[(size_t)(w2 * GI + g) * rec + Dh]);
      float L = 0.f, o[DPL];
#pragma unroll
      for (int d = 0; d < DPL; ++d) o[d] = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < kNWC; ++w2) {
        const float* src = sh + (size_t)(w2 * GI + g) * rec;
        const float lw = src[Dh + 1];
        const float wgt = lw > 0.f ? expf(src[Dh] - M) : 0.f;
        L += lw * wgt;
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[d] = fmaf(src[lane * DPL + d], wgt, o[d]);
      }
      const int h = hg * GI + g;
      const size_t oi = ((size_t)b * H + h) * Dh + lane * DPL;
      if (cph == 1) {
        const float invL = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
          const float v = X::rnd(o[d] * invL);
          if (st.flags & SF_OUT_T) X::st(st.out, oi + d, v);
          else reinterpret_cast<float*>(st.out)[oi + d] = v;
        }
      } else {
        // publish this CTA's part; the last of the cph CTAs merges the parts in part order
        const size_t pi = ((size_t)b * H + h) * cph + part;
#pragma unroll
        for (int d = 0; d < DPL; ++d) st.part_acc[pi * Dh + lane * DPL + d] = o[d];
        if (lane == 0) {
          st.part_ml[pi * 2 + 0] = M;
          st.part_ml[pi * 2 + 1] = L;
        }
        __threadfence();
        __syncwarp();
        int done = 0;
        if (lane == 0) done = atomicAdd(&st.counters[b * H + h], 1);
        done = __shfl_sync(0xffffffffu, done, 0);
        if (done == cph - 1) {
          __threadfence();
          const size_t hb = ((size_t)b * H + h) * cph;
          float pm[4], pl[4], pa[4][DPL];   // cph <= 4
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int c2 = min(c, cph - 1);
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(st.part_ml + (hb + c2) * 2));
            pm[c] = ml.x;
            pl[c] = ml.y;
            ld_row<float, DPL>(st.part_acc, (hb + c2) * Dh + lane * DPL, pa[c]);
          }
          float M2 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (c < cph) M2 = fmaxf(M2, pm[c]);
          float L2 = 0.f, o2[DPL];
#pragma unroll
          for (int d = 0; d < DPL; ++d) o2[d] = 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (c < cph) {
              const float wgt = pl[c] > 0.f ? expf(pm[c] - M2) : 0.f;
              L2 += pl[c] * wgt;
#pragma unroll
              for (int d = 0; d < DPL; ++d) o2[d] = fmaf(pa[c][d], wgt, o2[d]);
            }
          }
          const float invL = L2 > 0.f ? 1.f / L2 : 0.f;
#pragma unroll
          for (int d = 0; d < DPL; ++d) {
            const float v = X::rnd(o2[d] * invL);
            if (st.flags & SF_OUT_T) X::st(st.out, oi + d, v);
            else reinterpret_cast<float*>(st.out)[oi + d] = v;
          }
          if (lane == 0) st.counters[b * H + h] = 0;
        }
      }
    }
    cons_sync();   // the partial results in shared memory may be overwritten
  }
  if (!waited) barrier_wait(ab.sync, ab.giveup, ab.target, ab.s, tid);   // a CTA without items
}

template <typename T>
__device__ __forceinline__ void run_attn(const Stage& st, float* sh, const PosCache pc, const AttnBarrier ab) {
  const int G = qdiv(st.H, st.Hk);
  const int dpl = st.Dh / 32;
  if ((G & 1) == 0) {
    if (dpl == 4) attn_cta<T, 2, 4>(st, sh, pc, ab);
    else attn_cta<T, 2, 2>(st, sh, pc, ab);
  } else {
    if (dpl == 4) attn_cta<T, 1, 4>(st, sh, pc, ab);
    else attn_cta<T, 1, 2>(st, sh, pc, ab);
  }
}
// ----------------------------------------------------------------------------- small stages
template <typename T>
__device__ __forceinline__ void run_embed(const Stage& st, int gtid, int gthreads) {
  using X = TT<T>;
  const int d = st.P, B = st.B;
  for (int i = gtid; i < B * d; i += gthreads) {
    const int b = i / d, k = i - b * d;
    int tok = st.tokens[b];
    tok = min(max(tok, 0), st.vocab - 1);
    const float v = X::ld(st.WA, (size_t)tok * d + k);
    if (st.flags & SF_OUT_T) X::st(st.out, i, v);
    else reinterpret_cast<float*>(st.out)[i] = v;
  }
}

// CTA 0 only.  Lowest index wins among equal maxima.
static __device__ __forceinline__ void run_argmax(const Stage& st, float* redv, int* redi, int tid,
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
//   [.., +512)                  reduction scratch, the CTA's barrier arrival count, give-up flag
//   [.., +kSmallProgBytes)      copy of a by-value program (per-op launches)
//   [.., +512)                  ring mbarriers: full[kMaxSlots], empty[kMaxSlots]
//   -- header rounded to 1 KB --
//   [.., +nslots*slot_bytes)    the ring (8192-byte slots; 8704 when the program streams int4 tiles)
//   [.., +part_bytes)           partial sums of the warps (sized by the host for the program)
//   [.., +vec_bytes)            staged input vector, B rows of xstride elements
// Stage timeline (optional): trace[(s*grid + cta)*16 + k] = globaltimer at: 0 stage entry,
// 1 grid barrier passed, 2 vector staged, 3 stage done, 4 vector words arrived, 5 norm reduced,
// 7 boxes consumed.
template <typename T, bool Q4>
__global__ void __launch_bounds__(kThreads, 1)
fsvd_decode_kernel(const Stage* __restrict__ prog_global, const __grid_constant__ SmallProgram small,
                   const unsigned char* __restrict__ maps_global, const __grid_constant__ SmallMaps small_maps,
                   int use_small, int nstages, SyncState* sync, int xstride, int part_bytes,
                   int vec_bytes, int nslots, int slot_bytes, unsigned long long* trace, long long wait_limit) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  unsigned char* cur_base = smem;
  float* red = reinterpret_cast<float*>(smem + 2 * kStageBytesAl);
  int* flags_sh = reinterpret_cast<int*>(smem + 2 * kStageBytesAl + 256);
  Stage* small_sh = reinterpret_cast<Stage*>(smem + 2 * kStageBytesAl + 512);
  unsigned char* bars = smem + 2 * kStageBytesAl + 512 + kSmallProgBytes;
  unsigned char* ring = smem + smem_header_bytes();
  float* part = reinterpret_cast<float*>(ring + (size_t)nslots * (Q4 ? slot_bytes : kBoxBytes));
  char* xvec = reinterpret_cast<char*>(part) + part_bytes;
  volatile int* giveup = flags_sh + 1;

  Ring rg;
  rg.full = smem_u32(bars);
  rg.empty = rg.full + kMaxSlots * 8;
  rg.data = smem_u32(ring);
  rg.stride = (uint32_t)slot_bytes;
  rg.ns = nslots;

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
  // flags_sh[16..23]: positions of the batch rows, flags_sh[24..25]: the array they come from
  if (tid < 8) {
    // read the descriptors where they came from: the shared-memory copy is still being written
    const Stage* src = use_small ? small.st : prog_global;
    const int* sl = nullptr;
    for (int s = 0; s < nstages && !sl; ++s) sl = src[s].seqlens;
    int B0 = 0;
    if (sl) B0 = src[0].B;
    flags_sh[16 + tid] = (sl && tid < B0) ? sl[tid] : 0;
    if (tid == 0) *reinterpret_cast<const int**>(flags_sh + 24) = sl;
  }
  if (tid == 0) {
    flags_sh[0] = 0;   // warps of this CTA that have arrived at the pending grid barrier
    flags_sh[1] = 0;   // set when a wait ran out: nobody in this CTA waits again
    *reinterpret_cast<long long*>(flags_sh + 2) = wait_limit;
    for (int i = 0; i < nslots; ++i) {
      mbar_init(rg.full + i * 8, 1);
      mbar_init(rg.empty + i * 8, 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  constexpr int kStageWords = (int)(sizeof(Stage) / 4);
  __syncthreads();
  if (tid < kStageWords)
    reinterpret_cast<int*>(cur_base)[tid] = reinterpret_cast<const int*>(prog)[tid];

  unsigned nbar = 0;
  if (warp >= kNWC) {
    // ---------------- producers
    producer_loop<T, Q4>(prog, nstages, maps, rg, lane, sync, giveup);
  } else {
    // ---------------- consumers
    unsigned seq_base = 0;
    PosCache pc;
    pc.ptr = *reinterpret_cast<const int* const*>(flags_sh + 24);
    pc.pos = flags_sh + 16;
    for (int s = 0; s < nstages; ++s) {
      cons_sync();  // everybody is done with the previous stage's buffers; descriptor s landed
      const Stage& st = *reinterpret_cast<const Stage*>(cur_base + (s & 1) * kStageBytesAl);
      unsigned long long* trow =
          (trace && tid == 0) ? trace + ((size_t)s * gridDim.x + blockIdx.x) * 16 : nullptr;
      trace_mark(trow, 0);
      // the last consumer warp fetches the next descriptor while the others go on
      if (warp == kNWC - 1 && s + 1 < nstages) {
        int* dst = reinterpret_cast<int*>(cur_base + ((s + 1) & 1) * kStageBytesAl);
        const int* src = reinterpret_cast<const int*>(prog + s + 1);
        for (int i = lane; i < kStageWords; i += 32) dst[i] = src[i];
      }
      const unsigned long long target = (nbar + 1ull) * gridDim.x;
      if (st.flags & SF_BARRIER) ++nbar;
      if (st.type == ST_GEMV) {
        StageCtx cx;
        cx.s = s;
        cx.sync = sync;
        cx.bar_target = target;
        cx.xvec = xvec;
        cx.xstride = xstride;
        cx.red = red;
        cx.part = part;
        cx.ring = rg;
        cx.seq_base = seq_base;
        cx.giveup = giveup;
        cx.pc = pc;
        cx.trow = trow;
        seq_base += (unsigned)gemv_stage<T, Q4>(st, cx);
      } else {
        if (st.type == ST_ATTN) {
          AttnBarrier ab;
          ab.need = (st.flags & SF_BARRIER) != 0;
          ab.sync = sync;
          ab.giveup = giveup;
          ab.target = target;
          ab.s = s;
          run_attn<T>(st, part, pc, ab);
        } else {
          if (st.flags & SF_BARRIER) barrier_wait(sync, giveup, target, s, tid);
          trace_mark(trow, 1);
          if (st.type == ST_EMBED) {
            run_embed<T>(st, blockIdx.x * kConsThreads + tid, gridDim.x * kConsThreads);
          } else if (st.type == ST_ARGMAX) {
            if (blockIdx.x == 0) run_argmax(st, red, flags_sh + 8, tid, kConsThreads);
          }
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
  if (*giveup)
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  // The last CTA to finish zeroes the barrier count for the next launch (which counts its barriers
  // from zero, whatever its grid); every CTA has passed all its barriers before it can get here.
  if (tid == 0) {
    __threadfence();
    const unsigned done = atomicAdd(&sync->done_ctas, 1u);
    if (done == gridDim.x - 1) {
      sync->done_ctas = 0;
      sync->arrivals = 0;
      sync->launches += 1;
    }
  }
}

}  // namespace fsvd
