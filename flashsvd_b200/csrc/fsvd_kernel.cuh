// Persistent stage interpreter for single-token decode of low-rank (W = U·V) transformers.
//
// Launch geometry: one CTA per SM (cooperative launch), NW warps per CTA.  Every warp owns a
// private ring of ND shared-memory slots; a slot holds a tile of 4 factor rows x KC elements
// fetched with four `cp.async.bulk` copies that complete on the slot's mbarrier.  The fetch
// cursor of a warp walks the same deterministic item sequence as its compute cursor but runs
// up to ND tiles ahead, across stage boundaries, so the HBM stream does not drain while the
// CTAs synchronise between two dependent stages.
//
// All waits are bounded: a wait that runs out records an error code in SyncState::status and
// the kernel carries on without waiting again, so a fault in the protocol ends in an error
// return on the host, never in a hung device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "fsvd_stage.h"

namespace fsvd {

constexpr int kRowsPerTile = 4;
constexpr int kRowBytes = 1024;                      // bytes of one row piece inside a slot
constexpr int kSlotBytes = kRowsPerTile * kRowBytes; // 4 KB
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

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
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
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
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
};

// ----------------------------------------------------------------------------- cursors
// Geometry of a GEMV stage as the item walker needs it.
struct GemvGeom {
  const char* WA;
  const char* WB;
  int P, K, ldw, segs, kseg, rope_half, rot;
  int nkch;    // KC-chunks per full K segment
  int items;   // row groups x segments
};

struct Cursor {
  int s;    // stage index (nstages = exhausted)
  int it;   // item index inside the stage
  int j;    // tile index inside the item
  int nsub; // tiles of the current item
};

struct Tile {
  int p0;       // first logical row
  int g;        // operand group 0 = A, 1 = B
  int k0;       // first column
  int kc;       // columns in this tile
  int seg;      // K segment
};

template <typename T>
__device__ __forceinline__ void load_geom(const Stage* st, GemvGeom& g) {
  constexpr int KC = kRowBytes / (int)sizeof(T);
  g.WA = reinterpret_cast<const char*>(st->WA);
  g.WB = reinterpret_cast<const char*>(st->WB);
  g.P = st->P;
  g.K = st->K;
  g.ldw = st->ldw;
  g.segs = st->segs;
  g.kseg = st->kseg;
  g.rope_half = st->rope_half;
  g.rot = st->rot;
  g.nkch = (g.kseg + KC - 1) / KC;
  g.items = ((g.P + kRowsPerTile - 1) / kRowsPerTile) * g.segs;
}

template <typename T>
__device__ __forceinline__ int item_tiles(const GemvGeom& g, int it) {
  constexpr int KC = kRowBytes / (int)sizeof(T);
  const int seg = it % g.segs;
  const int klen = min(g.kseg, g.K - seg * g.kseg);
  const int n = (klen + KC - 1) / KC;
  return g.WB ? 2 * n : n;
}

template <typename T>
__device__ __forceinline__ void decode_tile(const GemvGeom& g, int it, int j, int nsub, Tile& t) {
  constexpr int KC = kRowBytes / (int)sizeof(T);
  const int grp = it / g.segs;
  t.seg = it - grp * g.segs;
  const int nk = g.WB ? (nsub >> 1) : nsub;
  t.g = (j >= nk) ? 1 : 0;
  const int kci = j - t.g * nk;
  const int kbeg = t.seg * g.kseg;
  const int kend = min(g.K, kbeg + g.kseg);
  t.k0 = kbeg + kci * KC;
  t.kc = min(KC, kend - t.k0);
  t.p0 = grp * kRowsPerTile;
}

__device__ __forceinline__ int phys_row(const GemvGeom& g, int p) {
  if (g.rope_half > 0) {
    const int h = p / g.rope_half;
    return h * 2 * g.rope_half + (p - h * g.rope_half);
  }
  return p;
}

// First item of this warp in a stage whose assignment is rotated by `rot`.
__device__ __forceinline__ int first_item(int wrank, int rot, int total_warps) {
  int f = wrank - rot;
  if (f < 0) f += total_warps;
  return f;
}

// ----------------------------------------------------------------------------- warp state
template <typename T, int ND, bool BULK>
struct WarpCtx {
  const Stage* prog;
  int nstages;
  int wrank, total_warps, lane;
  uint32_t ring;      // shared address of this warp's first slot
  uint32_t bars;      // shared address of this warp's first mbarrier
  const char* ring_ptr;
  unsigned fetch_seq, cons_seq;
  unsigned landed_seq;   // tiles [cons_seq, landed_seq) are known to have arrived
  unsigned max_inflight; // cap on fetch_seq - landed_seq: bounds the bytes this warp keeps queued
                         // in the memory system, and with it the latency of every other access
  Cursor fc;          // fetch cursor
  GemvGeom fg;        // geometry of the fetch cursor's stage
  SyncState* sync;
  unsigned long long* trow;  // trace row of (current stage, this CTA) for thread 0, else null
};

__device__ __forceinline__ void trace_mark(unsigned long long* trow, int k) {
  if (trow) trow[k] = gtimer();
}

// Position the cursor on the first item of the first GEMV stage at or after stage s.
template <typename T, int ND, bool BULK>
__device__ __forceinline__ void fetch_seek(WarpCtx<T, ND, BULK>& w, int s) {
  for (; s < w.nstages; ++s) {
    const Stage* st = w.prog + s;
    if (st->type != ST_GEMV) continue;
    load_geom<T>(st, w.fg);
    const int f = first_item(w.wrank, w.fg.rot, w.total_warps);
    if (f < w.fg.items) {
      w.fc.s = s;
      w.fc.it = f;
      w.fc.j = 0;
      w.fc.nsub = item_tiles<T>(w.fg, f);
      return;
    }
  }
  w.fc.s = w.nstages;
}

// Issue the bulk copies of as many tiles as the ring has free slots for.
template <typename T, int ND, bool BULK>
__device__ __forceinline__ void top_up(WarpCtx<T, ND, BULK>& w) {
  if (!BULK) return;
  while (w.landed_seq < w.fetch_seq &&
         mbar_test_wait(w.bars + (w.landed_seq % ND) * 8, (w.landed_seq / ND) & 1u))
    ++w.landed_seq;
  while (w.fc.s < w.nstages && (w.fetch_seq - w.cons_seq) < (unsigned)ND &&
         (w.fetch_seq - w.landed_seq) < w.max_inflight) {
    Tile t;
    decode_tile<T>(w.fg, w.fc.it, w.fc.j, w.fc.nsub, t);
    const int slot = w.fetch_seq % ND;
    const uint32_t bar = w.bars + slot * 8;
    const uint32_t dst = w.ring + slot * kSlotBytes;
    const int nrows = min(kRowsPerTile, w.fg.P - t.p0);
    const uint32_t row_bytes = (uint32_t)t.kc * (uint32_t)sizeof(T);
    if (w.lane == 0) {
      // The slot was last read through the generic proxy by this warp; order those reads
      // before the async-proxy writes of the new copies.
      fence_proxy_async_smem();
      mbar_expect_tx(bar, row_bytes * nrows);
    }
    __syncwarp();
    if (w.lane < nrows) {
      const char* base = t.g ? w.fg.WB : w.fg.WA;
      const size_t row = (size_t)phys_row(w.fg, t.p0) + w.lane;
      const char* src = base + (row * (size_t)w.fg.ldw + (size_t)t.k0) * sizeof(T);
      bulk_g2s(dst + w.lane * kRowBytes, src, row_bytes, bar);
    }
    ++w.fetch_seq;
    // advance the fetch cursor
    if (++w.fc.j == w.fc.nsub) {
      w.fc.j = 0;
      w.fc.it += w.total_warps;
      if (w.fc.it < w.fg.items) {
        w.fc.nsub = item_tiles<T>(w.fg, w.fc.it);
      } else {
        fetch_seek(w, w.fc.s + 1);
      }
    }
  }
}

template <typename T, int ND, bool BULK>
__device__ __forceinline__ void wait_slot(WarpCtx<T, ND, BULK>& w) {
  if (!BULK) return;
  const int slot = w.cons_seq % ND;
  const uint32_t parity = (w.cons_seq / ND) & 1u;
  const uint32_t bar = w.bars + slot * 8;
  if (!mbar_try_wait(bar, parity)) {
    const unsigned long long t0 = gtimer();
    while (!mbar_try_wait(bar, parity)) {
      if (gtimer() - t0 > kWaitLimitNs) {
        if (w.lane == 0) atomicCAS(&w.sync->status, DS_OK, DS_COPY_TIMEOUT);
        break;
      }
    }
  }
  if (w.landed_seq <= w.cons_seq) w.landed_seq = w.cons_seq + 1;
}

// Reduce acc[r] (r<4) over the warp.  Afterwards every lane holds the sum for row lane>>3.
__device__ __forceinline__ float reduce_rows4(const float* a, int lane) {
  const bool b4 = lane & 16, b3 = lane & 8;
  float keep0 = b4 ? a[2] : a[0];
  float keep1 = b4 ? a[3] : a[1];
  const float send0 = b4 ? a[0] : a[2];
  const float send1 = b4 ? a[1] : a[3];
  keep0 += __shfl_xor_sync(0xffffffffu, send0, 16);
  keep1 += __shfl_xor_sync(0xffffffffu, send1, 16);
  float k = b3 ? keep1 : keep0;
  const float s = b3 ? keep0 : keep1;
  k += __shfl_xor_sync(0xffffffffu, s, 8);
  k += __shfl_xor_sync(0xffffffffu, k, 4);
  k += __shfl_xor_sync(0xffffffffu, k, 2);
  k += __shfl_xor_sync(0xffffffffu, k, 1);
  return k;
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
__device__ __forceinline__ void st_tag(void* base, size_t i, float v, unsigned tag) {
  uint2 w2;
  w2.x = __float_as_uint(v);
  w2.y = tag;
  reinterpret_cast<uint2*>(base)[i] = w2;
}

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
      if (st.flags & SF_RESID_TAG) ax.a0 = __uint_as_float(__ldcg(reinterpret_cast<const uint2*>(st.resid) + i).x);
      else if (st.flags & SF_RESID_T) ax.a0 = X::ld(st.resid, i);
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
                                              float bsum, const EpiAux& ax, unsigned tag) {
  using X = TT<T>;
  const int P = st.P;
  switch (st.epi) {
    case EPI_PARTIAL: {
      const size_t i = ((size_t)seg * st.B + b) * P + p;
      if (st.flags & SF_OUT_TAG) st_tag(st.out, i, a, tag);
      else reinterpret_cast<float*>(st.out)[i] = a;
    } break;
    case EPI_STORE: {
      const float v = X::rnd(a);
      const size_t i = (size_t)b * P + p;
      if (st.flags & SF_OUT_T) X::st(st.out, i, v);
      else if (st.flags & SF_OUT_TAG) st_tag(st.out, i, v, tag);
      else reinterpret_cast<float*>(st.out)[i] = v;
    } break;
    case EPI_RESID: {
      const size_t i = (size_t)b * P + p;
      const float v = X::rnd(ax.a0 + X::rnd(a));
      if (st.flags & SF_OUT_T) X::st(st.out, i, v);
      else if (st.flags & SF_OUT_TAG) st_tag(st.out, i, v, tag);
      else reinterpret_cast<float*>(st.out)[i] = v;
    } break;
    case EPI_SWIGLU: {
      const float g = X::rnd(a), u = X::rnd(bsum);
      const float sg = X::rnd(g / (1.0f + expf(-g)));
      const float v = X::rnd(sg * u);
      const size_t i = (size_t)b * P + p;
      if (st.flags & SF_OUT_TAG) st_tag(st.out, i, v, tag);
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

template <typename T, int NB, int ND, bool BULK>
__device__ __forceinline__ void run_gemv(WarpCtx<T, ND, BULK>& w, const Stage& st,
                                         const char* xvec, int xstride, unsigned tag) {
  using X = TT<T>;
  constexpr int VEC = X::kVec;
  GemvGeom g;
  load_geom<T>(&st, g);
  const int lane = w.lane;
  const int B = st.B;

  for (int it = first_item(w.wrank, g.rot, w.total_warps); it < g.items; it += w.total_warps) {
    float acc[2][kRowsPerTile][NB];
#pragma unroll
    for (int gi = 0; gi < 2; ++gi)
#pragma unroll
      for (int r = 0; r < kRowsPerTile; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[gi][r][b] = 0.f;

    const int nsub = item_tiles<T>(g, it);
    Tile t;
    EpiAux ax;
    {
      const int p = (it / g.segs) * kRowsPerTile + (lane >> 3);
      const int b = lane & 7;
      if (b < B && p < g.P) epi_prefetch<T>(st, p, b, ax);
    }
    for (int j = 0; j < nsub; ++j) {
      top_up(w);
      decode_tile<T>(g, it, j, nsub, t);
      const int xoff = (t.g ? st.xB_off : st.xA_off) + t.k0;
      const char* wbase;
      size_t wstride;
      if (BULK) {
        wait_slot(w);
        if (j == 0) trace_mark(w.trow, 6);
        wbase = w.ring_ptr + (w.cons_seq % ND) * kSlotBytes;
        wstride = kRowBytes;
      } else {
        const char* base = t.g ? g.WB : g.WA;
        const int nrows_ok = min(kRowsPerTile, g.P - t.p0);
        (void)nrows_ok;
        wbase = base + ((size_t)phys_row(g, t.p0) * g.ldw + t.k0) * sizeof(T);
        wstride = (size_t)g.ldw * sizeof(T);
      }
      const int nrows = min(kRowsPerTile, g.P - t.p0);
      for (int c = lane * VEC; c < t.kc; c += 32 * VEC) {
        float xs[NB][VEC];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if (b < B) {
            const uint4 xv = *reinterpret_cast<const uint4*>(
                xvec + ((size_t)b * xstride + xoff + c) * sizeof(T));
            X::unpack(xv, xs[b]);
          } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) xs[b][e] = 0.f;
          }
        }
#pragma unroll
        for (int r = 0; r < kRowsPerTile; ++r) {
          uint4 wv;
          if (BULK) {
            wv = *reinterpret_cast<const uint4*>(wbase + r * wstride + (size_t)c * sizeof(T));
          } else {
            wv = (r < nrows) ? ld_nc_v4(wbase + r * wstride + (size_t)c * sizeof(T))
                             : make_uint4(0, 0, 0, 0);
          }
          float wf[VEC];
          X::unpack(wv, wf);
          if (t.g == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
              for (int e = 0; e < VEC; ++e) acc[0][r][b] = fmaf(wf[e], xs[b][e], acc[0][r][b]);
          } else {
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
              for (int e = 0; e < VEC; ++e) acc[1][r][b] = fmaf(wf[e], xs[b][e], acc[1][r][b]);
          }
        }
      }
      if (BULK) {
        __syncwarp();
        ++w.cons_seq;
      }
    }
    trace_mark(w.trow, 7);
    // item epilogue: lane (r*8 + b) finishes logical row p0+r of batch row b
    const bool hasB = g.WB != nullptr;
    const int r_own = lane >> 3;
    const int b_own = lane & 7;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float ta[kRowsPerTile], tb[kRowsPerTile];
#pragma unroll
      for (int r = 0; r < kRowsPerTile; ++r) {
        ta[r] = acc[0][r][b];
        tb[r] = acc[1][r][b];
      }
      const float sa = reduce_rows4(ta, lane);
      const float sb = hasB ? reduce_rows4(tb, lane) : 0.f;
      const int p = t.p0 + r_own;
      if (b_own == b && b < B && p < g.P) gemv_epilogue<T>(st, p, b, t.seg, sa, sb, ax, tag);
    }
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
// Bounded poll helper: returns true when the caller should give up.
struct SpinGuard {
  unsigned spins = 0;
  unsigned long long t0 = 0;
  __device__ __forceinline__ bool expired(SyncState* sync) {
    if ((++spins & 255u) != 0) return false;
    if (*reinterpret_cast<volatile int*>(&sync->status) != DS_OK) return true;
    const unsigned long long now = gtimer();
    if (t0 == 0) {
      t0 = now;
      return false;
    }
    if (now - t0 > kWaitLimitNs) {
      atomicCAS(&sync->status, DS_OK, DS_TAG_TIMEOUT);
      return true;
    }
    return false;
  }
};

// Polling load of two (value, tag) words.  Volatile so that the compiler re-issues it on every
// iteration of a spin loop; it is served by L2.
__device__ __forceinline__ uint4 ldcg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
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

// Brings the stage's input vector into shared memory as T.  All global loads of a thread are
// issued before the first use so that their L2 latencies overlap.  Tagged sources are polled
// until every word carries the tag of the producing stage.
template <typename T, int ND, bool BULK>
__device__ __noinline__ void stage_vector(WarpCtx<T, ND, BULK>& w, const Stage& st, char* xvec,
                                          int xstride, float* red, int tid, int nthreads,
                                          unsigned tag_base) {
  SyncState* sync = w.sync;
  using X = TT<T>;
  const int len = st.vl_len, B = st.B;
  const bool inT = (st.flags & SF_IN_T) != 0;
  const bool tagged = (st.flags & SF_IN_TAG) != 0;
  const unsigned want = tag_base + (unsigned)st.vl_tag + 1u;
  if (tagged && st.vl_mode == VL_SUM) {
    const int upr = len >> 1;  // 2-element units (one 16-byte load) per row
    const int units = B * upr;
    const int nseg = st.vl_nseg;
    const size_t segstride = (size_t)B * len * 8;  // bytes between partial sums
    const char* src = reinterpret_cast<const char*>(st.vl_src);
    if (nseg == 1) {
      constexpr int U = 8;
      for (int u0 = tid; u0 - (tid & 31) < units; u0 += nthreads * U) {  // warp-uniform trip count
        uint4 wv[U];
        SpinGuard sg;
        bool ok;
        do {
          ok = true;
#pragma unroll
          for (int q = 0; q < U; ++q) {
            const int u = u0 + q * nthreads;
            if (u < units) wv[q] = ldcg_u4(src + (size_t)u * 16);
          }
#pragma unroll
          for (int q = 0; q < U; ++q) {
            const int u = u0 + q * nthreads;
            if (u < units) ok = ok && wv[q].y == want && wv[q].w == want;
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) top_up(w);
        } while (!ok && !sg.expired(sync));
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = u0 + q * nthreads;
          if (u < units) {
            const int b = u / upr, k = (u - b * upr) * 2;
            st2<T>(xvec, (size_t)b * xstride + k, __uint_as_float(wv[q].x), __uint_as_float(wv[q].z));
          }
        }
      }
    } else {
      constexpr int SMAX = 8;  // kMaxSegs of the program builder
      for (int u = tid; u - (tid & 31) < units; u += nthreads) {  // warp-uniform trip count
        const bool act = u < units;
        uint4 wv[SMAX];
        SpinGuard sg;
        bool ok;
        do {
          ok = true;
#pragma unroll
          for (int q = 0; q < SMAX; ++q)
            if (act && q < nseg) wv[q] = ldcg_u4(src + q * segstride + (size_t)u * 16);
#pragma unroll
          for (int q = 0; q < SMAX; ++q)
            if (act && q < nseg) ok = ok && wv[q].y == want && wv[q].w == want;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) top_up(w);
        } while (!ok && !sg.expired(sync));
        if (act) {
          float a0 = __uint_as_float(wv[0].x), a1 = __uint_as_float(wv[0].z);
#pragma unroll
          for (int q = 1; q < SMAX; ++q)
            if (q < nseg) {
              a0 += __uint_as_float(wv[q].x);
              a1 += __uint_as_float(wv[q].z);
            }
          const int b = u / upr, k = (u - b * upr) * 2;
          st2<T>(xvec, (size_t)b * xstride + k, a0, a1);
        }
      }
    }
    return;
  }
  if (tagged && st.vl_mode == VL_RMSNORM) {
    constexpr int U = 8;
    const int upr = len >> 1;
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    const bool fits = upr <= nthreads * U;
    const char* src = reinterpret_cast<const char*>(st.vl_src);
    for (int b = 0; b < B; ++b) {
      const char* row = src + (size_t)b * len * 8;
      uint4 wv[U];
      float ss = 0.f;
      for (int u0 = tid; u0 - (tid & 31) < upr; u0 += nthreads * U) {  // warp-uniform trip count
        SpinGuard sg;
        bool ok;
        do {
          ok = true;
#pragma unroll
          for (int q = 0; q < U; ++q) {
            const int u = u0 + q * nthreads;
            if (u < upr) wv[q] = ldcg_u4(row + (size_t)u * 16);
          }
#pragma unroll
          for (int q = 0; q < U; ++q) {
            const int u = u0 + q * nthreads;
            if (u < upr) ok = ok && wv[q].y == want && wv[q].w == want;
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) top_up(w);
        } while (!ok && !sg.expired(sync));
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = u0 + q * nthreads;
          if (u < upr) {
            const float x0 = __uint_as_float(wv[q].x), x1 = __uint_as_float(wv[q].z);
            ss += x0 * x0 + x1 * x1;
          }
        }
      }
      trace_mark(w.trow, 4);
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int i = 0; i < nwarps; ++i) tot += red[i];
      const float inv = rsqrtf(tot / (float)len + st.eps);
      __syncthreads();
      trace_mark(w.trow, 5);
      auto finish = [&](int u, float x0, float x1) {
        float w0, w1;
        {
          float tmp[2];
          ld_row<T, 2>(st.vl_w, (size_t)u * 2, tmp);
          w0 = tmp[0];
          w1 = tmp[1];
        }
        st2<T>(xvec, (size_t)b * xstride + (size_t)u * 2, w0 * X::rnd(x0 * inv), w1 * X::rnd(x1 * inv));
      };
      if (fits) {
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = tid + q * nthreads;
          if (u < upr) finish(u, __uint_as_float(wv[q].x), __uint_as_float(wv[q].z));
        }
      } else {
        for (int u = tid; u < upr; u += nthreads) {
          const uint4 t = ldcg_u4(row + (size_t)u * 16);
          finish(u, __uint_as_float(t.x), __uint_as_float(t.z));
        }
      }
    }
    return;
  }
  const int upr = len >> 2;          // 4-element units per batch row
  const int units = B * upr;
  if (st.vl_mode == VL_SUM) {
    const int nseg = st.vl_nseg;
    const size_t segstride = (size_t)B * len;
    if (nseg == 1) {
      constexpr int U = 8;
      for (int u0 = tid; u0 < units; u0 += nthreads * U) {
        float4 v[U];
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = u0 + q * nthreads;
          if (u < units) v[q] = ld4<T>(st.vl_src, (size_t)u * 4, inT);
        }
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = u0 + q * nthreads;
          if (u < units) {
            const int b = u / upr, k = (u - b * upr) * 4;
            st4<T>(xvec, (size_t)b * xstride + k, v[q]);
          }
        }
      }
    } else {
      constexpr int SMAX = 8;  // kMaxSegs of the program builder
      for (int u = tid; u < units; u += nthreads) {
        float4 v[SMAX];
#pragma unroll
        for (int sgi = 0; sgi < SMAX; ++sgi)
          if (sgi < nseg) v[sgi] = ld4<T>(st.vl_src, sgi * segstride + (size_t)u * 4, inT);
        float4 a = v[0];
#pragma unroll
        for (int sgi = 1; sgi < SMAX; ++sgi)
          if (sgi < nseg) { a.x += v[sgi].x; a.y += v[sgi].y; a.z += v[sgi].z; a.w += v[sgi].w; }
        const int b = u / upr, k = (u - b * upr) * 4;
        st4<T>(xvec, (size_t)b * xstride + k, a);
      }
    }
  } else if (st.vl_mode == VL_RMSNORM) {
    constexpr int U = 8;  // register-resident units per thread; longer rows are re-read
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    const bool fits = upr <= nthreads * U;
    for (int b = 0; b < B; ++b) {
      float4 v[U];
      float ss = 0.f;
      if (fits) {
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = tid + q * nthreads;
          if (u < upr) v[q] = ld4<T>(st.vl_src, (size_t)b * len + (size_t)u * 4, inT);
        }
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = tid + q * nthreads;
          if (u < upr) ss += v[q].x * v[q].x + v[q].y * v[q].y + v[q].z * v[q].z + v[q].w * v[q].w;
        }
      } else {
        for (int u = tid; u < upr; u += nthreads) {
          const float4 t = ld4<T>(st.vl_src, (size_t)b * len + (size_t)u * 4, inT);
          ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
        }
      }
      trace_mark(w.trow, 4);
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int i = 0; i < nwarps; ++i) tot += red[i];
      const float inv = rsqrtf(tot / (float)len + st.eps);
      __syncthreads();
      trace_mark(w.trow, 5);
      auto finish = [&](int u, float4 t) {
        const float4 wv = ld4<T>(st.vl_w, (size_t)u * 4, true);
        t.x = wv.x * X::rnd(t.x * inv);
        t.y = wv.y * X::rnd(t.y * inv);
        t.z = wv.z * X::rnd(t.z * inv);
        t.w = wv.w * X::rnd(t.w * inv);
        st4<T>(xvec, (size_t)b * xstride + (size_t)u * 4, t);
      };
      if (fits) {
#pragma unroll
        for (int q = 0; q < U; ++q) {
          const int u = tid + q * nthreads;
          if (u < upr) finish(u, v[q]);
        }
      } else {
        for (int u = tid; u < upr; u += nthreads)
          finish(u, ld4<T>(st.vl_src, (size_t)b * len + (size_t)u * 4, inT));
      }
    }
  }
}

// ----------------------------------------------------------------------------- attention stage
// One item = (batch row, kv head, key split).  Lane l owns dims [l*DPL, (l+1)*DPL) of the head.
template <typename T, int G, int DPL>
__device__ __noinline__ void attn_items(const Stage& st, int wrank, int total_warps, int lane,
                                        unsigned tag) {
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
          else if (st.flags & SF_OUT_TAG) st_tag(st.out, oi + d, v, tag);
          else reinterpret_cast<float*>(st.out)[oi + d] = v;
        }
      }
      if (lane == 0) st.counters[b * Hk + hk] = 0;
    }
  }
}

template <typename T>
__device__ __forceinline__ void run_attn(const Stage& st, int wrank, int total_warps, int lane,
                                         unsigned tag) {
  const int G = st.H / st.Hk;
  const int dpl = st.Dh / 32;
#define FSVD_ATTN_CASE(GG, DD) \
  if (G == GG && dpl == DD) { attn_items<T, GG, DD>(st, wrank, total_warps, lane, tag); return; }
  FSVD_ATTN_CASE(1, 4)
  FSVD_ATTN_CASE(2, 4)
  FSVD_ATTN_CASE(4, 4)
  FSVD_ATTN_CASE(8, 4)
  FSVD_ATTN_CASE(1, 2)
  FSVD_ATTN_CASE(2, 2)
  FSVD_ATTN_CASE(4, 2)
  FSVD_ATTN_CASE(8, 2)
#undef FSVD_ATTN_CASE
}

// ----------------------------------------------------------------------------- small stages
template <typename T>
__device__ __noinline__ void run_embed(const Stage& st, int gtid, int gthreads, unsigned tag) {
  using X = TT<T>;
  const int d = st.P, B = st.B;
  for (int i = gtid; i < B * d; i += gthreads) {
    const int b = i / d, k = i - b * d;
    int tok = st.tokens[b];
    tok = min(max(tok, 0), st.vocab - 1);
    const float v = X::ld(st.WA, (size_t)tok * d + k);
    if (st.flags & SF_OUT_TAG) st_tag(st.out, i, v, tag);
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
}

// ----------------------------------------------------------------------------- the kernel
// Dynamic shared memory layout:
//   [0, NW*ND*8)                mbarriers
//   [.., +2*sizeof(Stage))      current and next stage descriptor
//   [.., +512)                  reduction scratch
//   [.., +kSmallProgBytes)      copy of a by-value program (per-op launches)
//   [.., +NW*ND*kSlotBytes)     rings (1024-byte aligned)
//   [.., +vec_bytes)            staged input vector, B rows of xstride elements
// Stage timeline (optional): trace[(s*grid + cta)*8 + k] = globaltimer at: 0 stage entry, 1 after
// the grid barrier, 2 vector staged, 3 body done (thread 0's warp), 4 vector words arrived,
// 5 norm reduced, 6 first tile of thread 0's warp landed, 7 last tile consumed.
template <typename T, int NB, int NW, int ND, bool BULK>
__global__ void __launch_bounds__(NW * 32, 1)
fsvd_decode_kernel(const Stage* __restrict__ prog_global, const __grid_constant__ SmallProgram small,
                   int use_small, int nstages, SyncState* sync, int xstride,
                   unsigned long long* trace, int max_inflight) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nthreads = NW * 32;

  constexpr int kBarBytes = ((NW * ND * 8 + 15) / 16) * 16;
  constexpr int kHdr = smem_header_bytes(NW, ND);
  unsigned char* cur_base = smem + kBarBytes;
  float* red = reinterpret_cast<float*>(smem + kBarBytes + 2 * kStageBytesAl);
  int* flags_sh = reinterpret_cast<int*>(smem + kBarBytes + 2 * kStageBytesAl + 256);
  Stage* small_sh = reinterpret_cast<Stage*>(smem + kBarBytes + 2 * kStageBytesAl + 512);
  unsigned char* rings = smem + kHdr;
  char* xvec = reinterpret_cast<char*>(rings + (BULK ? (size_t)NW * ND * kSlotBytes : 0));

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

  WarpCtx<T, ND, BULK> w;
  w.prog = prog;
  w.nstages = nstages;
  w.lane = lane;
  w.total_warps = gridDim.x * NW;
  w.wrank = warp * gridDim.x + blockIdx.x;
  w.ring = smem_u32(rings + (size_t)warp * ND * kSlotBytes);
  w.ring_ptr = reinterpret_cast<const char*>(rings + (size_t)warp * ND * kSlotBytes);
  w.bars = smem_u32(smem + warp * ND * 8);
  w.fetch_seq = 0;
  w.cons_seq = 0;
  w.landed_seq = 0;
  w.max_inflight = max_inflight > 0 ? (unsigned)max_inflight : (unsigned)ND;
  w.sync = sync;
  w.trow = nullptr;

  if (BULK) {
    if (lane == 0) {
      for (int i = 0; i < ND; ++i) mbar_init(w.bars + i * 8, 1);
      fence_mbar_init();
      fence_proxy_async_smem();
    }
    __syncwarp();
  }
  fetch_seek(w, 0);
  top_up(w);

  const unsigned long long bar_base = __ldcg(&sync->bar_base);
  const unsigned epoch = __ldcg(&sync->epoch);
  const unsigned tag_base = epoch * kTagStride;
  unsigned nbar = 0;
  constexpr int kStageWords = (int)(sizeof(Stage) / 4);

  // descriptor of stage 0
  if (tid < kStageWords)
    reinterpret_cast<int*>(cur_base)[tid] = reinterpret_cast<const int*>(prog)[tid];

  for (int s = 0; s < nstages; ++s) {
    __syncthreads();  // everybody is done with the previous stage's vector; descriptor s landed
    const Stage& st = *reinterpret_cast<const Stage*>(cur_base + (s & 1) * kStageBytesAl);
    if (trace && tid == 0) trace[((size_t)s * gridDim.x + blockIdx.x) * 8 + 0] = gtimer();
    w.trow = (trace && tid == 0) ? trace + ((size_t)s * gridDim.x + blockIdx.x) * 8 : nullptr;
    // the last warp fetches the next descriptor while the others go on
    if (warp == NW - 1 && s + 1 < nstages) {
      int* dst = reinterpret_cast<int*>(cur_base + ((s + 1) & 1) * kStageBytesAl);
      const int* src = reinterpret_cast<const int*>(prog + s + 1);
      for (int i = lane; i < kStageWords; i += 32) dst[i] = src[i];
    }
    if (st.flags & SF_BARRIER) {
      // Arrive once per CTA (the __syncthreads above ordered every warp's stores before it),
      // then every warp polls for itself and keeps its prefetch going meanwhile.
      if (tid == 0) {
        __threadfence();
        atomicAdd(&sync->arrivals, 1ull);
      }
      const unsigned long long target = (bar_base + nbar + 1ull) * gridDim.x;
      SpinGuard sg;
      bool ok;
      do {
        unsigned long long seen = 0;
        if (lane == 0) seen = ld_acquire_u64(&sync->arrivals);
        seen = __shfl_sync(0xffffffffu, seen, 0);
        ok = seen >= target;
        if (!ok) top_up(w);
      } while (!ok && !sg.expired(sync));
      if (!ok && tid == 0) sync->status_detail = s;
      __threadfence();
      ++nbar;
    }
    if (trace && tid == 0) trace[((size_t)s * gridDim.x + blockIdx.x) * 8 + 1] = gtimer();
    if (st.type == ST_GEMV) {
      if (st.vl_mode != VL_NONE) {
        stage_vector<T, ND, BULK>(w, st, xvec, xstride, red, tid, nthreads, tag_base);
        __syncthreads();
      }
      if (trace && tid == 0) trace[((size_t)s * gridDim.x + blockIdx.x) * 8 + 2] = gtimer();
      run_gemv<T, NB, ND, BULK>(w, st, xvec, xstride, tag_base + (unsigned)s + 1u);
    } else if (st.type == ST_ATTN) {
      run_attn<T>(st, w.wrank, w.total_warps, lane, tag_base + (unsigned)s + 1u);
    } else if (st.type == ST_EMBED) {
      run_embed<T>(st, blockIdx.x * nthreads + tid, gridDim.x * nthreads, tag_base + (unsigned)s + 1u);
    } else if (st.type == ST_ARGMAX) {
      if (blockIdx.x == 0) run_argmax(st, red, flags_sh, tid, nthreads);
    }
    top_up(w);
    if (trace && tid == 0) trace[((size_t)s * gridDim.x + blockIdx.x) * 8 + 3] = gtimer();
  }
  // The last CTA to finish publishes the barrier count and the next tag epoch; every CTA has
  // read both words before it can get here.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned done = atomicAdd(&sync->done_ctas, 1u);
    if (done == gridDim.x - 1) {
      sync->done_ctas = 0;
      sync->bar_base = bar_base + nbar;
      sync->epoch = epoch + 1u;
    }
  }
}

}  // namespace fsvd
