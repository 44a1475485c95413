// Persistent stage interpreter for single-token decode of low-rank (W = U·V) transformers.
//
// Launch geometry: one CTA per SM (cooperative launch), NW warps per CTA.  A GEMV stage is cut
// into units of 8 factor rows x one K segment; units go round-robin to the CTAs and inside a
// CTA the warps split the K range of every unit, so every warp of every SM streams factor bytes
// in every stage.  A lane loads its 16-byte fragment of a factor row straight from global
// memory into registers (ld.global.nc, D loads in flight per lane) and feeds it to the tensor
// cores; the partial sums of the warps meet in shared memory, are added in warp order and the
// stage's epilogue (RoPE + cache append, SiLU·up, residual, ...) runs on the result.
//
// The factors of a stage do not depend on the activations, so a warp issues its first D loads
// before it waits for the grid barrier in front of the stage, and prefetches the rows it will
// read in the following stage(s) into L2 (prefetch.global.L2): the HBM stream keeps running
// while the CTAs synchronise.
//
// (Measured on B200 before settling on this: per-warp shared-memory rings filled by
// cp.async.bulk stall the issuing warp ~320 cycles per copy and deliver after ~1 us; rings
// filled by 16-byte cp.async issue faster but still cost ~1700 cycles per 4 KB tile in issue,
// wait and shared-memory reads.  Direct loads cost ~10 instructions per 512 bytes and reach
// 6.5 TB/s with 8 warps x 16 loads in flight.)
//
// Arithmetic.  bf16: 8 factor rows x 32 columns are the B operand of two mma.sync.m16n8k16
// (fp32 accumulate) and the staged activation vector the A operand, batch rows as M.  A dot
// product does not care about the order of k, so lane (g, t) feeds the k-slots it owns with 8
// consecutive columns: one 16-byte load of factor row g and one of activation row g.  The four
// lanes of a quad cover 32 columns, the MMA adds them, and lane (g, t) holds the sums of
// factor rows 2t, 2t+1 for batch row g: no unpacking, no shuffles.  fp32 (parity mode): lane
// (g, t) multiplies 4 columns of row g with plain FMAs and the quad is reduced by shuffles.
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

constexpr int kTileRows = 8;
constexpr long long kWaitLimitClk = 4000000000ll;  // ~2 s of SM clocks

// ----------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
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
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
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
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Byte offset of 16-byte chunk `chunk` of row `row` inside a slot whose rows are RB bytes long.
template <int RB>
__device__ __forceinline__ uint32_t slot_off(int row, int chunk) {
  return (uint32_t)row * RB + (uint32_t)((chunk ^ ((row & 1) << 2)) << 4);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
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
};// ----------------------------------------------------------------------------- small helpers
__device__ __forceinline__ int phys_row(int rope_half, int p) {
  if (rope_half > 0) {
    const int h = p / rope_half;
    return h * 2 * rope_half + (p - h * rope_half);
  }
  return p;
}

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
struct EpiAux {
  float a0, a1;
  int pos;
};

template <typename T>
__device__ __forceinline__ void epi_prefetch(const Stage& st, int p, int b, EpiAux& ax) {
  using X = TT<T>;
  ax.a0 = ax.a1 = 0.f;
  ax.pos = 0;
  switch (st.epi) {
    case EPI_RESID: {
      const size_t i = (size_t)b * st.P + p;
      if (st.flags & SF_RESID_T) ax.a0 = X::ldcg(st.resid, i);
      else ax.a0 = __ldcg(reinterpret_cast<const float*>(st.resid) + i);
    } break;
    case EPI_ROPE_Q:
    case EPI_ROPE_K: {
      const int half = st.rope_half;
      const int j = p % half;
      ax.pos = st.seqlens[b];
      ax.a0 = X::ld(st.cos_tab, (size_t)ax.pos * half + j);
      ax.a1 = X::ld(st.sin_tab, (size_t)ax.pos * half + j);
    } break;
    case EPI_V:
      ax.pos = st.seqlens[b];
      break;
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
      const float v = X::rnd(ax.a0 + X::rnd(a));
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
      const int h = p / half, j = p - h * half;
      const int pos = ax.pos;
      const float c = ax.a0, sn = ax.a1;
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
        const size_t base = (((size_t)b * st.S_max + pos) * st.Hk + h) * st.Dh + j;
        X::st(st.cache, base, o1);
        X::st(st.cache, base + half, o2);
      }
    } break;
    case EPI_V: {
      const int pos = ax.pos;
      if (pos < st.S_max)
        X::st(st.cache, ((size_t)b * st.S_max + pos) * ((size_t)st.Hk * st.Dh) + p, X::rnd(a));
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
}// ----------------------------------------------------------------------------- vector stage-in
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
    // T -> T copy (nseg is 1 for every T source)
    constexpr int U = 4;
    const int upr = len / VEC, units = B * upr;
    for (int u0 = tid; u0 < units; u0 += nthreads * U) {
      uint4 v[U];
#pragma unroll
      for (int q = 0; q < U; ++q) {
        const int u = u0 + q * nthreads;
        if (u < units) v[q] = ld_raw16<T>(st.vl_src, (size_t)u * VEC);
      }
#pragma unroll
      for (int q = 0; q < U; ++q) {
        const int u = u0 + q * nthreads;
        if (u < units) {
          const int b = u / upr, k = (u - b * upr) * VEC;
          *reinterpret_cast<uint4*>(xvec + ((size_t)b * xstride + k) * sizeof(T)) = v[q];
        }
      }
    }
  } else if (st.vl_mode == VL_SUM) {
    // fp32 partial sums [nseg][B][len]
    constexpr int SMAX = 8;  // kMaxSegs of the program builder
    const int nseg = st.vl_nseg;
    const int upr = len >> 2, units = B * upr;
    const size_t segstride = (size_t)B * len;
    const float* src = reinterpret_cast<const float*>(st.vl_src);
    for (int u = tid; u < units; u += nthreads) {
      float4 v[SMAX];
#pragma unroll
      for (int q = 0; q < SMAX; ++q)
        if (q < nseg) v[q] = ldcg_f4(src + q * segstride + (size_t)u * 4);
      float4 a = v[0];
#pragma unroll
      for (int q = 1; q < SMAX; ++q)
        if (q < nseg) { a.x += v[q].x; a.y += v[q].y; a.z += v[q].z; a.w += v[q].w; }
      const int b = u / upr, k = (u - b * upr) * 4;
      st4<T>(xvec, (size_t)b * xstride + k, a);
    }
  } else if (st.vl_mode == VL_RMSNORM) {
    // T source, weight of type T; a row longer than the register window is read twice
    constexpr int U = 4;
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
      __syncthreads();
      float tot = 0.f;
      for (int i = 0; i < nwarps; ++i) tot += red[i];
      const float inv = rsqrtf(tot / (float)len + st.eps);
      __syncthreads();
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
}// ----------------------------------------------------------------------------- GEMV engine
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// The same load under a predicate; the registers are zero when it is off.  Written as one asm
// block: `pred ? load : 0` in C++ becomes a select on the loaded value, and the select makes the
// warp wait for the load, which serialises all loads in flight (measured ~800 cycles per load).
__device__ __forceinline__ uint4 ldg_stream_if(const void* p, bool pred) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.u32 q, %5, 0;\n\t"
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
      "@q ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
      : "=&r"(v.x), "=&r"(v.y), "=&r"(v.z), "=&r"(v.w)
      : "l"(p), "r"((unsigned)pred));
  return v;
}
// Refill of pipeline slot I while run `cur` is consumed (see gemv_stage): block b0 + I + D of
// the current run when it exists (I < r1 also says the lane's columns are inside the K range),
// else block I of the next run (I >= r2 and I < nl), else zeros.  Addresses are a base plus an
// immediate, the predicates compare round counters with immediates: no per-block arithmetic.
template <int I, int D>
__device__ __forceinline__ uint4 ldg_refill(const char* pb, const char* pn, int r1, int r2, int nl) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.gt.s32 p, %6, %9;\n\t"          // I < r1
      "setp.le.s32 q, %7, %9;\n\t"          // I >= r2
      "setp.gt.and.s32 q, %8, %9, q;\n\t"   // ... and I < nl
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
      "@p ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4+%10];\n\t"
      "@q ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%5+%11];\n\t}"
      : "=&r"(v.x), "=&r"(v.y), "=&r"(v.z), "=&r"(v.w)
      : "l"(pb), "l"(pn), "r"(r1), "r"(r2), "r"(nl), "n"(I), "n"((I + D) * 64), "n"(I * 64));
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
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// One unit of a GEMV stage as this CTA sees it: 8 logical rows x one K segment.
struct UnitInfo {
  unsigned long long row_off;  // byte offset of the unit's first factor row
  int p0, seg, kbeg, kend;
  int nblk;                    // blocks (one 16-byte load per lane each) in [kbeg, kend)
  int pad;
};
constexpr int kMaxUnitsPerCta = 64;

__device__ __forceinline__ void bulk_prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// L2 prefetch of the whole factor matrices of stage `st`: every warp of the grid asks for one
// contiguous share with a single bulk prefetch (per-line prefetches cost one LSU cycle per line,
// as much as the loads themselves).
template <typename T>
__device__ __forceinline__ void prefetch_stage(const Stage& st, int gwarp, int gwarps, int lane) {
  if (st.type != ST_GEMV || lane != 0) return;
  const size_t pitch = (size_t)st.ldw * sizeof(T);
  const size_t rows = st.rope_half > 0 ? (size_t)2 * st.P : (size_t)st.P;
  const size_t total = rows * pitch;                       // multiple of 16
  size_t share = (total / gwarps + 15) & ~(size_t)15;
  if (share < 2048) share = 2048;
  const size_t beg = (size_t)gwarp * share;
  if (beg >= total) return;
  const uint32_t n = (uint32_t)min(share, total - beg);
  bulk_prefetch_l2(reinterpret_cast<const char*>(st.WA) + beg, n);
  if (st.WB && st.rope_half == 0) bulk_prefetch_l2(reinterpret_cast<const char*>(st.WB) + beg, n);
}

// Grid barrier wait (one polling lane per CTA) in front of a stage with SF_BARRIER.
__device__ __forceinline__ void barrier_wait(SyncState* sync, unsigned long long target, int s, int tid) {
  if (tid == 0) {
    if (ld_acquire_u64(&sync->arrivals) < target) {
      const long long c0 = clock64();
      unsigned spins = 0;
      while (ld_acquire_u64(&sync->arrivals) < target) {
        if ((++spins & 63u) == 0) {
          if (*reinterpret_cast<volatile int*>(&sync->status) != DS_OK) break;
          if (clock64() - c0 > kWaitLimitClk) {
            atomicCAS(&sync->status, DS_OK, DS_BARRIER_TIMEOUT);
            sync->status_detail = s;
            break;
          }
        }
      }
    }
  }
  __syncthreads();
}

// Per-stage context handed to the stage functions.
struct StageCtx {
  const Stage* prog;
  int s, nstages;
  SyncState* sync;
  unsigned long long bar_target;   // arrival count that opens this stage's barrier
  char* xvec;
  int xstride;
  float* red;
  float* part;                     // partial sums: [unit ordinal][operand][k slice][batch 8][row 8]
  UnitInfo* units;                 // this CTA's units of the stage
  unsigned long long* trow;
};

// A run: the blocks one warp streams for one (unit, operand): its K slice of 8 factor rows.
// n / ui / g are warp-uniform, p / lim / xcol belong to the lane.
struct Run {
  const char* p;   // lane address of block 0 (factor row lane>>2, 16 bytes at column kcol)
  int n;           // blocks in the run; 0 = no more runs
  int lim;         // blocks whose 16 bytes of this lane lie inside the K range (ragged last block)
  int xcol;        // the lane's activation column for block 0, operand offset included
  int ui, g;       // unit ordinal of this CTA, operand group
};

template <typename T>
struct WarpGeo {
  const char* W[2];
  size_t pitch;
  int xoff[2];
  int nops, nu, P;
  int ks, kslice, slot, nslots;   // warps per unit, this warp's K slice and unit slot
  int qg, qt;
};

// Move `r` to the next (unit, operand) in which this warp owns blocks, starting the search at
// (ui, g).  Units are visited slot, slot + nslots, ...; operands 0, 1 inside a unit.
template <typename T>
__device__ __forceinline__ void run_seek(const WarpGeo<T>& wg, const UnitInfo* units, Run& r, int ui, int g) {
  constexpr int VEC = 16 / (int)sizeof(T), CB = 4 * VEC;
  for (; ui < wg.nu; ui += wg.nslots, g = 0) {
    const UnitInfo u = units[ui];
    const int bps = (u.nblk + wg.ks - 1) / wg.ks;
    const int j0 = wg.kslice * bps, j1 = min(u.nblk, j0 + bps);
    if (j0 >= j1) continue;
    // a row past the end of the matrix is replaced by the unit's first row; its sums land in
    // accumulator columns that are never stored
    const int row = (u.p0 + wg.qg < wg.P) ? wg.qg : 0;
    const int kcol = u.kbeg + j0 * CB + wg.qt * VEC;
    r.p = wg.W[g] + u.row_off + (size_t)row * wg.pitch + (size_t)kcol * sizeof(T);
    r.n = j1 - j0;
    r.lim = max(0, min(r.n, (u.kend - kcol + CB - 1) / CB));
    r.xcol = wg.xoff[g] + kcol;
    r.ui = ui;
    r.g = g;
    return;
  }
  r.n = 0;
  r.lim = 0;
  r.ui = wg.nu;
  r.g = 0;
}
template <typename T>
__device__ __forceinline__ void run_next(const WarpGeo<T>& wg, const UnitInfo* units, const Run& cur, Run& nxt) {
  if (cur.n == 0) {
    nxt = cur;
    return;
  }
  if (cur.g + 1 < wg.nops) run_seek<T>(wg, units, nxt, cur.ui, cur.g + 1);
  else run_seek<T>(wg, units, nxt, cur.ui + wg.nslots, 0);
}

// One GEMV stage, all warps of the CTA.
//
// Register pipeline: every run is padded to whole rounds of D blocks and slot s of buf[] holds
// the block with index % D == s, so every index into buf[] is a compile-time constant and a
// slot is always refilled with the block D ahead in the padded stream: block b + D of the run
// being consumed or, in its last round, block s of the next run.
template <typename T, int NW, int D>
__device__ __noinline__ void gemv_stage(const Stage& st, const StageCtx& cx) {
  using X = TT<T>;
  constexpr int VEC = 16 / (int)sizeof(T), CB = 4 * VEC;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nthreads = NW * 32;
  const int B = st.B;
  const int grid = gridDim.x;

  const long long k0 = clock64();
  // ---- 0. this CTA's units of the stage, computed once into shared memory
  const int total_units = ((st.P + kTileRows - 1) / kTileRows) * st.segs;
  const int first = first_item(blockIdx.x, st.rot % grid, grid);
  const int nu = first < total_units ? min(kMaxUnitsPerCta, (total_units - first + grid - 1) / grid) : 0;
  if (tid < nu) {
    const int uidx = first + tid * grid;
    UnitInfo u;
    const int grp = uidx / st.segs;
    u.seg = uidx - grp * st.segs;
    u.p0 = grp * kTileRows;
    u.kbeg = u.seg * st.kseg;
    u.kend = min(st.K, u.kbeg + st.kseg);
    u.nblk = (u.kend - u.kbeg + CB - 1) / CB;
    u.row_off = (unsigned long long)phys_row(st.rope_half, u.p0) * st.ldw * sizeof(T);
    u.pad = 0;
    cx.units[tid] = u;
  }
  __syncthreads();

  const long long k1 = clock64();
  WarpGeo<T> wg;
  wg.W[0] = reinterpret_cast<const char*>(st.WA);
  wg.W[1] = reinterpret_cast<const char*>(st.WB);
  wg.pitch = (size_t)st.ldw * sizeof(T);
  wg.xoff[0] = st.xA_off;
  wg.xoff[1] = st.xB_off;
  wg.nops = st.WB ? 2 : 1;
  wg.nu = nu;
  wg.P = st.P;
  wg.ks = st.ksplit > 0 ? st.ksplit : NW;
  wg.kslice = warp % wg.ks;
  wg.slot = warp / wg.ks;
  wg.nslots = NW / wg.ks;
  wg.qg = lane >> 2;
  wg.qt = lane & 3;
  const UnitInfo* units = cx.units;

  // operands of the epilogues this thread will run (outputs tid and tid + nthreads), fetched
  // now so that their latency hides behind the streaming
  const int nout = nu * kTileRows * B;
  EpiAux ax0, ax1;
  ax0.a0 = ax0.a1 = ax1.a0 = ax1.a1 = 0.f;
  ax0.pos = ax1.pos = 0;
  auto out_pos = [&](int o, int& i, int& b, int& r) {
    i = o / (kTileRows * B);
    const int rem = o - i * (kTileRows * B);
    b = rem / kTileRows;
    r = rem - b * kTileRows;
  };
  {
    int i, b, r;
    if (tid < nout) {
      out_pos(tid, i, b, r);
      const int p = cx.units[i].p0 + r;
      if (p < st.P) epi_prefetch<T>(st, p, b, ax0);
    }
    if (tid + nthreads < nout) {
      out_pos(tid + nthreads, i, b, r);
      const int p = cx.units[i].p0 + r;
      if (p < st.P) epi_prefetch<T>(st, p, b, ax1);
    }
  }
  // ---- 1. first loads of this warp, before any waiting
  Run cur, nxt;
  run_seek<T>(wg, units, cur, wg.slot, 0);
  run_next<T>(wg, units, cur, nxt);
  uint4 buf[D];
#pragma unroll
  for (int s = 0; s < D; ++s) buf[s] = ldg_stream_if(cur.p + s * 64, s < cur.lim);
  const long long k2 = clock64();
  // ---- 2. L2 prefetch of the stages the host assigned to this one
  for (int t = st.pf_begin; t < st.pf_end; ++t)
    prefetch_stage<T>(cx.prog[t], warp * grid + blockIdx.x, grid * NW, lane);

  const long long k3 = clock64();
  // ---- 3. wait for the producers of the input vector, stage it
  if (st.flags & SF_BARRIER) barrier_wait(cx.sync, cx.bar_target, cx.s, tid);
  trace_mark(cx.trow, 1);
  if (st.vl_mode != VL_NONE) {
    stage_vector<T>(st, cx.xvec, cx.xstride, cx.red, tid, nthreads, cx.trow);
    __syncthreads();
  }
  trace_mark(cx.trow, 2);

  const long long k4 = clock64();
  // ---- 4. stream this warp's runs
  const bool xact = wg.qg < B;
  const uint32_t xvec_s = smem_u32(cx.xvec);
  const uint32_t xlane_s = xvec_s + (uint32_t)(xact ? wg.qg : 0) * cx.xstride * (uint32_t)sizeof(T);
  const uint32_t xrow_bytes = (uint32_t)cx.xstride * (uint32_t)sizeof(T);
  while (cur.n > 0) {
    float acc[2][4];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[c][e] = 0.f;
    const char* pb = cur.p;                  // lane address of block b0
    const char* pn = nxt.p;
    // activation bytes of block b0 for this lane; blocks past `lim` multiply zeros, their
    // activation loads may run up to one block past the K range (the host pads the vector)
    uint32_t xs = (sizeof(T) == 2 ? xlane_s : xvec_s) + (uint32_t)cur.xcol * (uint32_t)sizeof(T);
    // A run is padded to a whole number of rounds of D blocks (the padding blocks load nothing
    // and multiply zeros), so the block D ahead of block b0 + I is block b0 + I + D of this run
    // or, in the last round, block I of the next one.
    const int np = (cur.n + D - 1) / D * D;
    int r1 = cur.lim - D, r2 = np - D;       // I < r1: own block b0+I+D holds data; I >= r2: next run's turn
    const int nl = nxt.lim;

    auto consume = [&](auto iconst, const uint4& wv) {
      constexpr int I = decltype(iconst)::value;
      if constexpr (sizeof(T) == 2) {
        const uint4 xv = lds128_imm<I * 64>(xs);
        mma_bf16_16816(acc[I & 1], xv.x, 0u, xv.y, 0u, wv.x, wv.y);
        mma_bf16_16816(acc[(I & 1) ^ 1], xv.z, 0u, xv.w, 0u, wv.z, wv.w);
      } else {
        // fp32: 4 columns of factor row qg times activation rows 0..3; acc[0][b] per batch row
        float wf[4], xf[4];
        X::unpack(wv, wf);
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) {
          if (bb < B) {
            const uint4 xb = lds128_imm<I * 64>(xs + bb * xrow_bytes);
            X::unpack(xb, xf);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[0][bb] = fmaf(wf[e], xf[e], acc[0][bb]);
          }
        }
      }
    };
    for (int left = np; left > 0; left -= D) {
      [&]<int... I>(std::integer_sequence<int, I...>) {
        ((void)([&] {
           const uint4 wv = buf[I];
           buf[I] = ldg_refill<I, D>(pb, pn, r1, r2, nl);
           consume(std::integral_constant<int, I>{}, wv);
         }()),
         ...);
      }(std::make_integer_sequence<int, D>{});
      pb += D * 64;
      xs += D * 64;
      r1 -= D;
      r2 -= D;
    }
    // publish the partial sums of this run
    {
      float* dst = cx.part + ((size_t)(cur.ui * wg.nops + cur.g) * wg.ks + wg.kslice) * 64;
      if constexpr (sizeof(T) == 2) {
        // lane (qg, qt): batch row qg, factor rows 2qt, 2qt+1
        if (xact) {
          dst[wg.qg * 8 + 2 * wg.qt] = acc[0][0] + acc[1][0];
          dst[wg.qg * 8 + 2 * wg.qt + 1] = acc[0][1] + acc[1][1];
        }
      } else {
        // quad reduction: lanes (qg, 0..3) hold 4 columns each of factor row qg
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) {
          float v = acc[0][bb];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if (wg.qt == bb && bb < B) dst[bb * 8 + wg.qg] = v;
        }
      }
    }
    cur = nxt;
    run_next<T>(wg, units, cur, nxt);
  }
  trace_mark(cx.trow, 7);
  const long long k5 = clock64();
  __syncthreads();
  const long long k6 = clock64();

  // ---- 5. add the slices' partial sums in slice order and run the epilogue
  for (int o = tid, it = 0; o < nout; o += nthreads, ++it) {
    int i, b, r;
    out_pos(o, i, b, r);
    const UnitInfo u = units[i];
    const int p = u.p0 + r;
    if (p >= st.P) continue;
    EpiAux ax;
    if (it == 0) ax = ax0;
    else if (it == 1) ax = ax1;
    else epi_prefetch<T>(st, p, b, ax);
    const int bps = (u.nblk + wg.ks - 1) / wg.ks;
    const int nsl = (u.nblk + bps - 1) / bps;   // slices that own blocks of this unit
    float sum[2] = {0.f, 0.f};
    for (int g = 0; g < wg.nops; ++g) {
      const float* src = cx.part + ((size_t)(i * wg.nops + g) * wg.ks) * 64 + b * 8 + r;
      float a = 0.f;
      for (int w2 = 0; w2 < nsl; ++w2) a += src[w2 * 64];
      sum[g] = a;
    }
    gemv_epilogue<T>(st, p, b, u.seg, sum[0], sum[1], ax);
  }
  if (cx.trow) {
    cx.trow[8] = k1 - k0;
    cx.trow[9] = k2 - k1;
    cx.trow[10] = k3 - k2;
    cx.trow[11] = k4 - k3;
    cx.trow[12] = k5 - k4;
    cx.trow[13] = k6 - k5;
    cx.trow[14] = clock64() - k6;
    cx.trow[15] = wg.ks;
  }
}

// ----------------------------------------------------------------------------- attention stage
// One item = (batch row, kv head, key split).  Lane l owns dims [l*DPL, (l+1)*DPL) of the head.
template <typename T, int G, int DPL>
__device__ __noinline__ void attn_items(const Stage& st, int wrank, int total_warps, int lane) {
  using X = TT<T>;
  constexpr int UNR = (G * DPL >= 16) ? 4 : 8;  // keys in flight per warp, bounded by registers
  const int Dh = st.Dh, Hk = st.Hk, H = st.H, nsplit = st.nsplit, B = st.B;
  const int items = B * Hk * nsplit;
  const size_t kv_row = (size_t)Hk * Dh;
  const bool qT = (st.flags & SF_IN_T) != 0;

  for (int it = first_item(wrank, st.rot, total_warps); it < items; it += total_warps) {
    const int sp = it % nsplit;
    const int hk = (it / nsplit) % Hk;
    const int b = it / (nsplit * Hk);
    const int n = min(st.seqlens[b] + st.seqlen_add, st.S_max);
    const int per = (n + nsplit - 1) / nsplit;
    const int j0 = sp * per, j1 = min(n, j0 + per);

    float q[G][DPL], acc[G][DPL], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const size_t qi = ((size_t)b * H + hk * G + g) * Dh + lane * DPL;
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
    const size_t base = ((size_t)b * st.S_max) * kv_row + (size_t)hk * Dh + lane * DPL;
    for (int j = j0; j < j1; j += UNR) {
      float kf[UNR][DPL], vf[UNR][DPL];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int jj = min(j + u, j1 - 1);
        ld_row<T, DPL>(st.kcache, base + (size_t)jj * kv_row, kf[u]);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int jj = min(j + u, j1 - 1);
        ld_row<T, DPL>(st.vcache, base + (size_t)jj * kv_row, vf[u]);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        if (j + u < j1) {
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float s = 0.f;
#pragma unroll
            for (int d = 0; d < DPL; ++d) s = fmaf(q[g][d], kf[u][d], s);
            s = warp_sum(s) * st.scale;
            const float mn = fmaxf(m[g], s);
            const float corr = expf(m[g] - mn);
            const float p = expf(s - mn);
            l[g] = l[g] * corr + p;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[g][d] = fmaf(p, vf[u][d], acc[g][d] * corr);
            m[g] = mn;
          }
        }
      }
    }
    // publish the partial result of this split
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const size_t pi = (((size_t)b * H + hk * G + g) * nsplit + sp);
#pragma unroll
      for (int d = 0; d < DPL; ++d) st.part_acc[pi * Dh + lane * DPL + d] = acc[g][d];
      if (lane == 0) {
        st.part_ml[pi * 2 + 0] = m[g];
        st.part_ml[pi * 2 + 1] = l[g];
      }
    }
    __threadfence();
    __syncwarp();
    int done = 0;
    if (lane == 0) done = atomicAdd(&st.counters[b * Hk + hk], 1);
    done = __shfl_sync(0xffffffffu, done, 0);
    if (done == nsplit - 1) {
      // Last split of this (b, kv head) to arrive: combine all splits in split order, whoever
      // the last arriver is, so the result does not depend on timing.  nsplit <= 32: lane s
      // fetches the (max, sum) pair of split s.
      __threadfence();
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const size_t hb = ((size_t)b * H + hk * G + g) * nsplit;
        float ms = -INFINITY, ls = 0.f;
        if (lane < nsplit) {
          const float2 ml = __ldcg(reinterpret_cast<const float2*>(st.part_ml + (hb + lane) * 2));
          ms = ml.x;
          ls = ml.y;
        }
        const float M = warp_max(ms);
        const float wgt = ls > 0.f ? expf(ms - M) : 0.f;
        float L = 0.f, o[DPL];
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[d] = 0.f;
        for (int s0 = 0; s0 < nsplit; s0 += 8) {
          float pa[8][DPL];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int s2 = min(s0 + u, nsplit - 1);
            ld_row<float, DPL>(st.part_acc, (hb + s2) * Dh + lane * DPL, pa[u]);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int s2 = min(s0 + u, 31);
            const float ws = __shfl_sync(0xffffffffu, wgt, s2);
            const float lw = __shfl_sync(0xffffffffu, ls, s2) * ws;
            if (s0 + u < nsplit) {
              L += lw;
#pragma unroll
              for (int d = 0; d < DPL; ++d) o[d] = fmaf(pa[u][d], ws, o[d]);
            }
          }
        }
        const float invL = L > 0.f ? 1.f / L : 0.f;
        const size_t oi = ((size_t)b * H + hk * G + g) * Dh + lane * DPL;
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
          const float v = X::rnd(o[d] * invL);
          if (st.flags & SF_OUT_T) X::st(st.out, oi + d, v);
          else reinterpret_cast<float*>(st.out)[oi + d] = v;
        }
      }
      if (lane == 0) st.counters[b * Hk + hk] = 0;
    }
  }
}

template <typename T>
__device__ __forceinline__ void run_attn(const Stage& st, int wrank, int total_warps, int lane) {
  const int G = st.H / st.Hk;
  const int dpl = st.Dh / 32;
#define FSVD_ATTN_CASE(GG, DD) \
  if (G == GG && dpl == DD) { attn_items<T, GG, DD>(st, wrank, total_warps, lane); return; }
  FSVD_ATTN_CASE(1, 4)
  FSVD_ATTN_CASE(2, 4)
  FSVD_ATTN_CASE(4, 4)
  FSVD_ATTN_CASE(8, 4)
  FSVD_ATTN_CASE(1, 2)
  FSVD_ATTN_CASE(2, 2)
  FSVD_ATTN_CASE(4, 2)
  FSVD_ATTN_CASE(8, 2)
#undef FSVD_ATTN_CASE
}// ----------------------------------------------------------------------------- small stages
template <typename T>
__device__ __noinline__ void run_embed(const Stage& st, int gtid, int gthreads) {
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
static __device__ __noinline__ void run_argmax(const Stage& st, float* redv, int* redi, int tid,
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
    __syncthreads();
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
    __syncthreads();
  }
  if (tid == 0) *st.step_counter = step + 1;
}// ----------------------------------------------------------------------------- the kernel
// Dynamic shared memory layout:
//   [0, 2*sizeof(Stage))        current and next stage descriptor
//   [.., +512)                  reduction scratch and the CTA's barrier arrival count
//   [.., +kSmallProgBytes)      copy of a by-value program (per-op launches)
//   [.., +kMaxUnitsPerCta*32)   this CTA's units of the running stage
//   [.., +part_bytes)           partial sums of the warps (sized by the host for the program)
//   [.., +vec_bytes)            staged input vector, B rows of xstride elements
// Stage timeline (optional): trace[(s*grid + cta)*16 + k] = globaltimer at: 0 stage entry,
// 1 grid barrier passed, 2 vector staged, 3 stage done, 4 vector words arrived, 5 norm reduced,
// 7 blocks streamed.
template <typename T, int NW, int D>
__global__ void __launch_bounds__(NW * 32, 1)
fsvd_decode_kernel(const Stage* __restrict__ prog_global, const __grid_constant__ SmallProgram small,
                   int use_small, int nstages, SyncState* sync, int xstride, int part_bytes,
                   int vec_bytes, unsigned long long* trace) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nthreads = NW * 32;

  unsigned char* cur_base = smem;
  float* red = reinterpret_cast<float*>(smem + 2 * kStageBytesAl);
  int* flags_sh = reinterpret_cast<int*>(smem + 2 * kStageBytesAl + 256);
  Stage* small_sh = reinterpret_cast<Stage*>(smem + 2 * kStageBytesAl + 512);
  UnitInfo* units = reinterpret_cast<UnitInfo*>(smem + 2 * kStageBytesAl + 512 + kSmallProgBytes);
  static_assert(sizeof(UnitInfo) == 32, "unit table entry size");
  float* part = reinterpret_cast<float*>(smem + smem_header_bytes());
  char* xvec = reinterpret_cast<char*>(smem + smem_header_bytes() + part_bytes);

  // Padding blocks of a run multiply zero factors with whatever follows the K range in the
  // staged vector, so that memory must hold finite numbers from the start.
  for (int i = tid; i < vec_bytes / 16; i += nthreads)
    reinterpret_cast<uint4*>(xvec)[i] = make_uint4(0, 0, 0, 0);

  const Stage* prog = prog_global;
  if (use_small) {
    // by-value program: copy it to shared memory once and walk it there
    const int* src = reinterpret_cast<const int*>(small.st);
    int* dst = reinterpret_cast<int*>(small_sh);
    const int nwords = nstages * (int)(sizeof(Stage) / 4);
    for (int i = tid; i < nwords; i += nthreads) dst[i] = src[i];
    prog = small_sh;
    __syncthreads();
  }
  const int wrank = warp * gridDim.x + blockIdx.x, total_warps = gridDim.x * NW;

  const unsigned long long bar_base = __ldcg(&sync->bar_base);
  unsigned nbar = 0;
  constexpr int kStageWords = (int)(sizeof(Stage) / 4);
  // flags_sh[0]: warps of this CTA that have arrived at the pending grid barrier
  if (tid == 0) flags_sh[0] = 0;
  if (tid < kStageWords)
    reinterpret_cast<int*>(cur_base)[tid] = reinterpret_cast<const int*>(prog)[tid];

  for (int s = 0; s < nstages; ++s) {
    __syncthreads();  // everybody is done with the previous stage's buffers; descriptor s landed
    const Stage& st = *reinterpret_cast<const Stage*>(cur_base + (s & 1) * kStageBytesAl);
    unsigned long long* trow =
        (trace && tid == 0) ? trace + ((size_t)s * gridDim.x + blockIdx.x) * 16 : nullptr;
    trace_mark(trow, 0);
    // the last warp fetches the next descriptor while the others go on
    if (warp == NW - 1 && s + 1 < nstages) {
      int* dst = reinterpret_cast<int*>(cur_base + ((s + 1) & 1) * kStageBytesAl);
      const int* src = reinterpret_cast<const int*>(prog + s + 1);
      for (int i = lane; i < kStageWords; i += 32) dst[i] = src[i];
    }
    const unsigned long long target = (bar_base + nbar + 1ull) * gridDim.x;
    if (st.flags & SF_BARRIER) ++nbar;
    if (st.type == ST_GEMV) {
      StageCtx cx;
      cx.prog = prog;
      cx.s = s;
      cx.nstages = nstages;
      cx.sync = sync;
      cx.bar_target = target;
      cx.xvec = xvec;
      cx.xstride = xstride;
      cx.red = red;
      cx.part = part;
      cx.units = units;
      cx.trow = trow;
      gemv_stage<T, NW, D>(st, cx);
    } else {
      if (st.flags & SF_BARRIER) barrier_wait(sync, target, s, tid);
      trace_mark(trow, 1);
      if (st.type == ST_ATTN) {
        run_attn<T>(st, wrank, total_warps, lane);
      } else if (st.type == ST_EMBED) {
        run_embed<T>(st, blockIdx.x * nthreads + tid, gridDim.x * nthreads);
      } else if (st.type == ST_ARGMAX) {
        if (blockIdx.x == 0) run_argmax(st, red, flags_sh + 8, tid, nthreads);
      }
    }
    if (st.flags & SF_ARRIVE) {
      // Grid-barrier arrival, warp by warp: each warp publishes its own stores and counts itself
      // in shared memory; the last warp of the CTA adds the CTA to the global count.
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        unsigned old;
        asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;"
                     : "=r"(old) : "r"(smem_u32(flags_sh)) : "memory");
        if (old == (unsigned)NW - 1u) {
          flags_sh[0] = 0;
          asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(&sync->arrivals) : "memory");
        }
      }
    }
    trace_mark(trow, 3);
  }
  // The last CTA to finish publishes the barrier count for the next launch; every CTA has read
  // it before it can get here.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned done = atomicAdd(&sync->done_ctas, 1u);
    if (done == gridDim.x - 1) {
      sync->done_ctas = 0;
      sync->bar_base = bar_base + nbar;
    }
  }
}

}  // namespace fsvd
