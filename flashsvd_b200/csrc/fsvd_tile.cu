// Decode for batches of 9..128 sequences (bf16): the factor products as tiled GEMMs on the 5th
// generation tensor cores.
//
// With more than 8 activation rows per factor row the 16 x 8 register tiles of the persistent
// interpreter (fsvd_kernel.cuh) no longer fit the batch; here a factor product is
//     D[128 factor rows, N batch columns] = W[128, K] . X[N, K]^T        (N = batch rounded up to 16)
// issued as tcgen05.mma (cta_group::1, kind::f16, M = 128) by one thread per CTA, with both operands
// read from shared memory (128-byte swizzled, K-major, filled by TMA) and the fp32 accumulator in
// tensor memory.  The work is still bound by the factor stream from HBM (each factor byte is used
// for N <= 128 multiply-adds), so the kernel is organised around keeping TMA busy:
//   * one CTA = one tile of 128 factor rows x one K segment; the <= 8 segments of a tile are the CTAs
//     of a thread-block cluster: they exchange their partial sums through distributed shared memory
//     (each CTA finishes a slice of the batch columns, adding the segments in segment order), so
//     no partial sum goes through global memory and the result does not depend on timing;
//   * a ring of NS stages {W tile 16 KB, (second W tile), X tile(s)}: three threads issue the TMA copies
//     as slots free up, thread 32 issues the MMAs as slots fill and releases a slot with
//     tcgen05.commit, all four warps read the accumulator back with tcgen05.ld for the epilogue;
//   * epilogues: store / residual / SwiGLU (two accumulators) / RoPE + q buffer / RoPE + key cache /
//     value cache, with the rounding points of the PyTorch low-rank path (every nn.Linear output
//     rounded to bf16), the same as the interpreter's.
// A decoder layer is 12 launches on the caller's stream (2 RMSNorm, 9 GEMM launches over its 13
// factors with the q / k / v lifts grouped, attention with the split merge inside the kernel); a
// model step is captured once into a CUDA graph.  Attention: batch_attn_kernel (1 or 2 query heads per
// kv head, shuffle-reduced dot products at the HBM rate), gqa_decode_attn_kernel (4 or 8: the heads as
// rows of a tensor-core tile), prompt_attn_kernel (causal attention of a prompt pass).
// Tensor-parallel layer (fsvd_tile_tp_decode_layer): the o lift and the down lift end in the push
// epilogue (TE_PUSH: partial sums stored into every rank's exchange region over peer memory, one flag
// per CTA), exchange_reduce_rows_kernel sums them in rank order with the residual and applies the
// RMSNorm that follows; protocol in fsvd_exchange.h.
//
// Reference functions replaced: kernels/mlp/decode/dual_split_triton_pcat_s.py:39-120 (token-tiled
// SwiGLU MLP), kernels/attn/decode/densekv_reconstruct_triton.py:464-760 (q/k/v lift),
// runtime/attn/decode_registry.py:177-211 (rotary + append + attention), for batches > 8.
//
// Every wait in these kernels is bounded (clock64 budget); a wait that runs out sets the status word,
// the CTA frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/flashsvd_b200.h"
#include "fsvd_exchange.h"
#include "fsvd_stage.h"
#include "fsvd_tile.h"

namespace fsvd_tile {

using fsvd::DS_BARRIER_TIMEOUT;
using fsvd::DS_CACHE_FULL;
using fsvd::DS_COPY_TIMEOUT;
using fsvd::DS_OK;
using fsvd::SyncState;

constexpr int kTileM = 128;          // factor rows of a tile (UMMA M)
constexpr int kTileK = 64;           // bf16 elements of a k-block: one 128-byte swizzle span
constexpr int kThreads = 128;        // 4 warps: warp w reads accumulator lanes 32 w .. 32 w + 31
constexpr int kWTileBytes = kTileM * kTileK * 2;   // 16 KB
constexpr int kMaxStages = 8;
constexpr int kMaxSegs = 8;           // K segments of a tile = CTAs of a cluster (portable size)

enum TileEpi : int {
  TE_STORE = 0,      // out[b, p] = rnd(acc)                        (bf16)
  TE_STORE_F32 = 1,  // out[b, p] = rnd(acc) kept in an fp32 container (logits)
  TE_RESID = 2,      // out[b, p] = rnd(resid[b, p] + rnd(acc))
  TE_SWIGLU = 3,     // out[b, p] = rnd(rnd(silu(rnd(accA))) * rnd(accB))      A = gate, B = up
  TE_ROPE_Q = 4,     // rotate the head's (j, j + Dh/2) pair at position seqlens[b], store to out[b, p]
  TE_ROPE_K = 5,     // same rotation, store into the key cache at position seqlens[b]
  TE_VCACHE = 6,     // store rnd(acc) into the value cache at position seqlens[b]
  TE_PUSH = 7,       // tensor-parallel partial sums: rnd(acc) into this rank's slot of every rank's exchange region
};

struct GemmArgs {
  int P, K, B, N;          // factor rows, reduction length, batch rows, batch rounded up to 16
  int tiles, segs, kbs;    // row tiles, K segments, k-blocks per segment
  int nkb;                 // k-blocks in all
  int nstages, two, epi;
  uint32_t tmem_cols;      // power of two >= 32
  int cpo;                 // batch columns finished by each CTA of a tile's cluster: ceil(N / segs) rounded up to 4
  void* out;
  const void* resid;
  void* cache;             // TE_ROPE_K / TE_VCACHE: [rows, S_max, Hk, Dh]
  const void* cos_tab;
  const void* sin_tab;
  const int* seqlens;
  int Dh, HkDh, S_max, shared_cache;
  int* status;             // SyncState::status of the workspace
  long long wait_limit;
  unsigned long long* trace;   // debugging: %globaltimer marks, 16 per CTA (null = off)
  fsvd_exch::Geom ex;          // TE_PUSH: the exchange regions of all ranks (fsvd_exchange.h)
  const unsigned* ex_seq;      // TE_PUSH: this rank's exchange sequence number
};

// ------------------------------------------------------------------------------- PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tma_box_2d(uint32_t dst, const void* tmap, int col, int row, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(col), "r"(row), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]^T, one 128 x N x 16 step
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has finished
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 16 consecutive accumulator columns of this thread's lane
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor: K-major tile of rows x 64 bf16, 128-byte swizzle (the layout a
// TMA box of 64 columns with CU_TENSOR_MAP_SWIZZLE_128B leaves): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128, N.
__device__ __forceinline__ uint32_t umma_idesc(int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}

// Cluster barrier (all threads of all CTAs of the cluster) and a store into the shared memory of
// the cluster's CTA `rank` at the same offset as the local address `addr`.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t rank, float x, float y, float z, float w) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

__device__ __forceinline__ void tmark(const GemmArgs& a, int k) {
  if (a.trace && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    a.trace[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + k] = t;
  }
}

__device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float ldbf(const void* p, size_t i) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void stbf(void* p, size_t i, float v) {
  reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Bounded mbarrier wait; false when the budget ran out or the CTA has given up already.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* giveup, const GemmArgs& a, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*giveup) return false;
  const long long c0 = clock64();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0) {
      if (*giveup) return false;
      if (clock64() - c0 > a.wait_limit) {
        atomicCAS(a.status, (int)DS_OK, code);
        *giveup = 1;
        return false;
      }
    }
  }
  return true;
}

// Programmatic dependent launch: every kernel of this file is launched with the stream-serialization
// attribute, so its CTAs may start while the kernel before it in the stream is still draining.
// pdl_wait() returns when that kernel has completed and its writes are visible; nothing that
// another kernel wrote is read, and nothing in global memory is written, before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Up to three independent GEMMs in one launch (the q, k and v lifts of a layer): blockIdx.z picks
// the problem, CTAs outside a problem's (tiles, segs) range leave at once.
constexpr int kMaxGroup = 3;
struct GemmGroup {
  CUtensorMap maps[kMaxGroup][4];   // A, A2, X, X2
  GemmArgs args[kMaxGroup];
};

// ------------------------------------------------------------------------------- GEMM kernel
// grid = (tiles, segs, problems).  Dynamic shared memory: [1 KB slack for alignment][NS stages].
__global__ void __launch_bounds__(kThreads) tile_gemm_kernel(const __grid_constant__ GemmGroup grp) {
  const GemmArgs& a = grp.args[blockIdx.z];
  if ((int)blockIdx.x >= a.tiles || (int)blockIdx.y >= a.segs) return;
  const CUtensorMap& mapA = grp.maps[blockIdx.z][0];
  const CUtensorMap& mapA2 = grp.maps[blockIdx.z][1];
  const CUtensorMap& mapX = grp.maps[blockIdx.z][2];
  const CUtensorMap& mapX2 = grp.maps[blockIdx.z][3];
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * kMaxStages + 1];
  __shared__ uint32_t tmem_slot;
  __shared__ int giveup_sh;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, seg = blockIdx.y;
  tmark(a, 0);
  const int N = a.N, NS = a.nstages;
  const uint32_t xbytes = (uint32_t)N * 128u;
  const uint32_t stage_bytes = (uint32_t)kWTileBytes * (a.two ? 2u : 1u) + xbytes * (a.two ? 2u : 1u);
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kMaxStages]), accum = smem_u32(&bars[2 * kMaxStages]);
  volatile int* giveup = &giveup_sh;

  if (tid == 0) {
    giveup_sh = 0;
    for (int i = 0; i < NS; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, 1);
    }
    mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    tc_alloc(smem_u32(&tmem_slot), a.tmem_cols);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  tmark(a, 1);
  pdl_launch_dependents();

  const int kb0 = seg * a.kbs, kb1 = min(a.nkb, kb0 + a.kbs);
  const int nit = kb1 - kb0;

  if (warp != 1) {
    if (lane == 0) {
      // ---- producers: TMA copies of the stage operands.  One thread sustains about 24 GB/s of
      // copies (wait, arm, issue per box), so three threads (warps 0, 2, 3) share the stages.  A
      // ring slot always belongs to the same thread (slot % 3): a parity wait cannot tell phase k of
      // a slot's barrier from phase k + 2, and only a slot's single owner, which visits its rounds in
      // order, can never be two phases behind.
      // The factor tiles of the first NS stages do not depend on the kernel before this one and
      // are requested before pdl_wait().
      const int pj = warp == 0 ? 0 : warp - 1;
      constexpr int kProducers = 3;
      const int pre = min(nit, NS);
      for (int it = 0; it < pre; ++it) {
        if (it % kProducers != pj) continue;
        const uint32_t fb = full0 + 8 * it;
        const uint32_t dst = base + (uint32_t)it * stage_bytes;
        const int kcol = (kb0 + it) * kTileK;
        mbar_expect_tx(fb, stage_bytes);
        tma_box_2d(dst, &mapA, kcol, tile * kTileM, fb);
        if (a.two) tma_box_2d(dst + kWTileBytes, &mapA2, kcol, tile * kTileM, fb);
      }
      pdl_wait();
      for (int it = 0; it < nit; ++it) {
        const int s = it % NS, round = it / NS;
        if (s % kProducers != pj) continue;
        if (round > 0 && !wait_bar(empty0 + 8 * s, (uint32_t)(round - 1) & 1u, giveup, a, DS_COPY_TIMEOUT)) break;
        const uint32_t fb = full0 + 8 * s;
        uint32_t dst = base + (uint32_t)s * stage_bytes;
        const int kcol = (kb0 + it) * kTileK;
        if (it >= pre) {
          mbar_expect_tx(fb, stage_bytes);
          tma_box_2d(dst, &mapA, kcol, tile * kTileM, fb);
          if (a.two) tma_box_2d(dst + kWTileBytes, &mapA2, kcol, tile * kTileM, fb);
        }
        dst += (uint32_t)kWTileBytes * (a.two ? 2u : 1u);
        tma_box_2d(dst, &mapX, kcol, 0, fb);
        if (a.two) tma_box_2d(dst + xbytes, &mapX2, kcol, 0, fb);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issue: four 16-deep steps per k-block and accumulator.  The first activation tile
      // cannot arrive before the kernel in front has completed: the wait budget starts there.
      const uint32_t idesc = umma_idesc(N);
      bool ok = true;
      pdl_wait();
      for (int it = 0; it < nit && ok; ++it) {
        const int s = it % NS, round = it / NS;
        ok = wait_bar(full0 + 8 * s, (uint32_t)round & 1u, giveup, a, DS_COPY_TIMEOUT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = base + (uint32_t)s * stage_bytes;
        const uint32_t sx = sa + (uint32_t)kWTileBytes * (a.two ? 2u : 1u);
        const uint64_t da = umma_desc(sa), dx = umma_desc(sx);
#pragma unroll
        for (int kk = 0; kk < kTileK / 16; ++kk)
          tc_mma(tmem, da + 2u * kk, dx + 2u * kk, idesc, (it > 0 || kk > 0) ? 1u : 0u);
        if (a.two) {
          const uint64_t da2 = umma_desc(sa + kWTileBytes), dx2 = umma_desc(sx + xbytes);
#pragma unroll
          for (int kk = 0; kk < kTileK / 16; ++kk)
            tc_mma(tmem + (uint32_t)N, da2 + 2u * kk, dx2 + 2u * kk, idesc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(empty0 + 8 * s);   // the slot is free when these MMAs have read it
      }
      if (ok) tc_commit(accum);      // the accumulators are complete
    }
    __syncwarp();
  }

  // ---- everybody: wait for the kernel before this one (the epilogue reads what it wrote), then
  // for the accumulators
  pdl_wait();
  tmark(a, 2);
  const unsigned push_seq = a.epi == TE_PUSH ? *reinterpret_cast<const volatile unsigned*>(a.ex_seq) : 0u;
  // the residual rows this CTA will add have usually left L2 since they were written (a layer's
  // factors stream through in between): ask for them now, the epilogue is several microseconds away
  if (a.epi == TE_RESID && lane == 0) {
    const int prow = tile * kTileM + warp * 32;
    if (prow < a.P)
      for (int sl = 0; sl < a.cpo; ++sl) {
        const int b = seg * a.cpo + sl;
        if (b < a.B)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const __nv_bfloat16*>(a.resid) + (size_t)b * a.P + prow));
      }
  }
  bool have = nit > 0 ? wait_bar(accum, 0u, giveup, a, DS_BARRIER_TIMEOUT) : false;
  have = __all_sync(0xffffffffu, have);
  tc_fence_after();
  tmark(a, 3);

  const int r = tid;                       // accumulator lane = row of the tile
  const int p = tile * kTileM + r;         // factor row
  const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
  const int nacc = a.two ? 2 : 1;
  const int cpo = a.cpo;                   // batch columns finished by each CTA of the cluster

  // ---- the K segments of a tile are the CTAs of one cluster (rank = segment).  CTA j finishes the
  // batch columns [j cpo, (j + 1) cpo) (cpo a multiple of 4): every CTA sends its partial sums of
  // those columns to CTA j's shared memory, [accumulator][segment][row][cpo] floats, four columns per
  // 16-byte store; the ring is free for that once every CTA of the cluster has its accumulators
  // (first cluster barrier), and the sums are complete after the second.  Every CTA reaches both
  // barriers, whatever happened before.
  float* recv = reinterpret_cast<float*>(base_ptr);
  const uint32_t recv_u32 = base;
  cluster_sync();
  tmark(a, 4);
  if (have) {
    for (int acc = 0; acc < nacc; ++acc) {
      for (int c0 = 0; c0 < N; c0 += 16) {
        float v[16];
        tc_ld16(trow + (uint32_t)(acc * N + c0), v);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int col = c0 + 4 * q4;
          const int owner = col / cpo, slot = col - owner * cpo;
          if (owner < a.segs)
            st_cluster_v4(recv_u32 + (uint32_t)(((((acc * a.segs + seg) * kTileM + r) * cpo) + slot) * 4), (uint32_t)owner,
                          v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
        }
      }
    }
  }
  tmark(a, 5);
  cluster_sync();
  tmark(a, 6);

  if (!*giveup && have && p < a.P) {
    const int half = a.Dh >> 1;
    const bool rope = a.epi == TE_ROPE_Q || a.epi == TE_ROPE_K;
    const int j = rope ? p % a.Dh : 0;
    const bool lower = !rope || j < half;      // RoPE: the thread of row j < Dh/2 finishes rows j and j + Dh/2
    for (int sl = 0; sl < cpo && lower; sl += 4) {
      const int b0 = seg * cpo + sl;
      if (b0 >= a.B) break;
      // sums over the segments, in segment order, of four columns (and of the second accumulator,
      // or of the RoPE partner row)
      float v[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
      for (int sg = 0; sg < a.segs; ++sg) {
        const float4 t = *reinterpret_cast<const float4*>(recv + ((size_t)(sg * kTileM + r) * cpo + sl));
        v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
      }
      if (a.two || rope) {
        for (int sg = 0; sg < a.segs; ++sg) {
          const size_t row2 = a.two ? (size_t)((a.segs + sg) * kTileM + r) : (size_t)(sg * kTileM + r + half);
          const float4 t = *reinterpret_cast<const float4*>(recv + (row2 * cpo + sl));
          u[0] += t.x; u[1] += t.y; u[2] += t.z; u[3] += t.w;
        }
      }
      // One compact code path per epilogue kind (this code runs once per CTA, from a cold
      // instruction cache: the fewer lines it spans, the sooner it is through); within a kind the
      // operands of the four columns are loaded first, then come the arithmetic and the stores.
      const int nb = min(4, a.B - b0);
      const size_t o0 = (size_t)b0 * a.P + p;
      if (a.epi == TE_STORE) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < nb) stbf(a.out, o0 + (size_t)i * a.P, v[i]);
      } else if (a.epi == TE_RESID) {
        float res[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) res[i] = ldbf(a.resid, o0 + (size_t)min(i, nb - 1) * a.P);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < nb) stbf(a.out, o0 + (size_t)i * a.P, res[i] + rnd(v[i]));
      } else if (a.epi == TE_PUSH) {
        // the same rounded partial sums into slot [parity][this rank] of every rank's region
        // (peer stores over NVLink; the rank's own region among them)
        for (int q = 0; q < a.ex.world; ++q) {
          unsigned char* dst = fsvd_exch::slot_ptr(a.ex, q, push_seq & 1u, a.ex.rank);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (i < nb) stbf(dst, o0 + (size_t)i * a.P, v[i]);
        }
      } else if (a.epi == TE_SWIGLU) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float g = rnd(v[i]), up = rnd(u[i]);
          const float sg = rnd(g / (1.0f + expf(-g)));
          if (i < nb) stbf(a.out, o0 + (size_t)i * a.P, sg * up);
        }
      } else if (a.epi == TE_STORE_F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < nb) reinterpret_cast<float*>(a.out)[o0 + (size_t)i * a.P] = rnd(v[i]);
      } else {
        // value cache / rotary epilogues: position of every column, tables, then the stores
        int pos[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) pos[i] = a.seqlens[min(b0 + i, a.B - 1)];
        float cs[4], sn[4];
        if (rope) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int pt = min(pos[i], a.S_max - 1);
            cs[i] = ldbf(a.cos_tab, (size_t)pt * half + j);
            sn[i] = ldbf(a.sin_tab, (size_t)pt * half + j);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int b = b0 + i;
          if (i >= nb) continue;
          if (pos[i] >= a.S_max && a.epi != TE_ROPE_Q) {
            atomicCAS(a.status, (int)DS_OK, (int)DS_CACHE_FULL);
            continue;
          }
          const size_t oc = ((size_t)(a.shared_cache ? 0 : b) * a.S_max + pos[i]) * (size_t)a.HkDh + p;
          if (a.epi == TE_VCACHE) {
            stbf(a.cache, oc, v[i]);
          } else {
            const float x1 = rnd(v[i]), x2 = rnd(u[i]);
            const float o1 = rnd(rnd(x1 * cs[i]) - rnd(x2 * sn[i]));
            const float o2 = rnd(rnd(x2 * cs[i]) + rnd(x1 * sn[i]));
            if (a.epi == TE_ROPE_Q) {
              stbf(a.out, o0 + (size_t)i * a.P, o1);
              stbf(a.out, o0 + (size_t)i * a.P + half, o2);
            } else {
              stbf(a.cache, oc, o1);
              stbf(a.cache, oc + half, o2);
            }
          }
        }
      }
    }
  }

  // ---- release the tensor memory
  tmark(a, 7);
  tc_fence_before();
  __syncthreads();
  // TE_PUSH: every store of this CTA is ordered before the flags that thread q raises in rank q's
  // region: the CTA barrier above, then a store with release semantics at system scope (it orders the
  // writes the thread has observed through the barrier as well as its own)
  if (a.epi == TE_PUSH && tid < a.ex.world) {
    fsvd_exch::st_release_sys(fsvd_exch::flag_ptr(a.ex, tid, push_seq & 1u, a.ex.rank, tile * a.segs + seg), push_seq);
  }
  __syncwarp();
  if (*giveup)
    for (int i = 0; i < 100; ++i) __nanosleep(1000);   // copies in flight towards this CTA land first
  if (warp == 0) tc_dealloc(tmem, a.tmem_cols);
  tmark(a, 8);
}

// ------------------------------------------------------------------------------- RMSNorm rows
// out[b, :] = rnd(w * rnd(x[b, :] * rsqrt(mean(x[b, :]^2) + eps))), one CTA per row.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ out, int d, float eps) {
  __shared__ float red[8];
  const int b = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const __nv_bfloat16* xr = x + (size_t)b * d;
  float ss = 0.0f;
  for (int i = tid; i < d; i += 256) {
    const float v = __bfloat162float(xr[i]);
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)d + eps);
  for (int i = tid; i < d; i += 256)
    out[(size_t)b * d + i] = __float2bfloat16_rn(__bfloat162float(w[i]) * rnd(__bfloat162float(xr[i]) * inv));
}

// ------------------------------------------------------------------------------- exchange + RMSNorm rows
// Second half of a tensor-parallel exchange (protocol: fsvd_exchange.h).  Row b is shared by the
// gridDim.y CTAs of a cluster, each with a slice of its columns:
//     wait until every rank's GEMM has posted exchange number seq in this rank's region,
//     h[b, :]  = rnd(resid[b, :] + rnd(sum over ranks, in rank order, of slot[rank][b, :]))
//     xn[b, :] = rnd(w * rnd(h[b, :] * rsqrt(mean(h[b, :]^2) + eps)))             (when xn != null)
// The slots are read past L1 (another GPU wrote them); the CTAs of a row exchange their sums of
// squares through distributed shared memory and add them in CTA order.  The last CTA of the grid to
// finish advances the rank's sequence number.  A wait that runs out records DS_PEER_TIMEOUT and the
// rank it waited for; the row is then computed from whatever the slots hold.
struct ReduceArgs {
  fsvd_exch::Geom ex;
  fsvd_exch::Ctrl* ctrl;
  int nflags;                    // CTAs of the pushing GEMM
  const __nv_bfloat16* resid;
  __nv_bfloat16* out;
  const __nv_bfloat16* norm_w;
  __nv_bfloat16* xn;
  int d;
  float eps;
  int* status;                   // SyncState::status, status_detail of the workspace
  long long wait_limit;
  unsigned long long* trace;     // optional: record [seq % trace_cap] = %globaltimer at {dependency met, all flags seen, done}
  unsigned trace_cap;            // (written by CTA (0, 0))
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

__global__ void __launch_bounds__(256) exchange_reduce_rows_kernel(const __grid_constant__ ReduceArgs a) {
  __shared__ float red[8];
  __shared__ float css[kMaxSegs];            // sums of squares of the row's column slices
  __shared__ int giveup_sh;
  const int b = blockIdx.x, tid = threadIdx.x;
  const int C = gridDim.y, c = blockIdx.y;    // C > 1: launched as clusters of C CTAs along y
  if (tid == 0) giveup_sh = 0;
  pdl_launch_dependents();
  pdl_wait();
  __syncthreads();
  volatile int* giveup = &giveup_sh;
  const unsigned seq = *reinterpret_cast<const volatile unsigned*>(&a.ctrl->seq);
  const unsigned par = seq & 1u;
  unsigned long long* rec = (a.trace && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) ? a.trace + (size_t)(seq % a.trace_cap) * 3 : nullptr;
  if (rec) rec[0] = global_ns();
  {
    const int total = a.ex.world * a.nflags;
    const long long c0 = clock64();
    for (int i = tid; i < total && !*giveup; i += 256) {
      const int src = i / a.nflags;
      const unsigned* f = fsvd_exch::flag_ptr(a.ex, a.ex.rank, par, src, i - src * a.nflags);
      unsigned spins = 0;
      while ((int)(fsvd_exch::ld_acquire_sys(f) - seq) < 0) {
        if ((++spins & 15u) == 0) {
          if (*giveup) break;
          if (clock64() - c0 > a.wait_limit) {
            if (atomicCAS(a.status, (int)DS_OK, (int)fsvd_exch::DS_PEER_TIMEOUT) == (int)DS_OK) a.status[1] = src;
            *giveup = 1;
            break;
          }
        }
      }
    }
  }
  __syncthreads();
  if (rec) rec[1] = global_ns();
  if (C > 1 && a.xn) cluster_sync();            // every CTA of the row runs before any writes into its shared memory

  const int cols = a.d / C, col0 = c * cols;    // the host makes cols a multiple of 8
  const size_t row = (size_t)b * a.d + col0;
  const unsigned char* slot0 = fsvd_exch::slot_ptr(a.ex, a.ex.rank, par, 0);
  float ss = 0.0f;
  for (int i = tid * 8; i < cols; i += 256 * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (int q = 0; q < a.ex.world; ++q) {
      const uint4 t = __ldcg(reinterpret_cast<const uint4*>(slot0 + (size_t)q * a.ex.slot_bytes + (row + i) * 2));
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f2 = __bfloat1622float2(h2[j]);
        acc[2 * j] += f2.x;
        acc[2 * j + 1] += f2.y;
      }
    }
    const uint4 rr = *reinterpret_cast<const uint4*>(a.resid + row + i);
    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f2 = __bfloat1622float2(r2[j]);
      const float h0 = rnd(f2.x + rnd(acc[2 * j])), h1 = rnd(f2.y + rnd(acc[2 * j + 1]));
      ss += h0 * h0 + h1 * h1;
      o2[j] = __floats2bfloat162_rn(h0, h1);
    }
    *reinterpret_cast<uint4*>(a.out + row + i) = o;
  }
  if (a.xn) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    if (C > 1) {
      if (tid < C) st_cluster_f32(smem_u32(&css[c]), (uint32_t)tid, tot);
      cluster_sync();
      tot = 0.0f;
      for (int j = 0; j < C; ++j) tot += css[j];
    }
    const float inv = rsqrtf(tot / (float)a.d + a.eps);
    for (int i = tid * 8; i < cols; i += 256 * 8) {
      // the thread reads back the eight values it stored above
      const uint4 hh = *reinterpret_cast<const uint4*>(a.out + row + i);
      const uint4 ww = *reinterpret_cast<const uint4*>(a.norm_w + col0 + i);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hh);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&ww);
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 hf = __bfloat1622float2(h2[j]), wf = __bfloat1622float2(w2[j]);
        o2[j] = __floats2bfloat162_rn(wf.x * rnd(hf.x * inv), wf.y * rnd(hf.y * inv));
      }
      *reinterpret_cast<uint4*>(a.xn + row + i) = o;
    }
  }
  // every CTA has read the sequence number before it arrives here: the last one moves it on
  __syncthreads();
  if (rec) rec[2] = global_ns();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(&a.ctrl->done, 1u) == gridDim.x * gridDim.y - 1) {
      a.ctrl->done = 0u;
      *reinterpret_cast<volatile unsigned*>(&a.ctrl->seq) = seq + 1u;
    }
  }
}

// ------------------------------------------------------------------------------- attention
// Single-query attention of B sequences over their dense caches.  One CTA = (sequence, kv head,
// key split); its G = H / Hk query heads share the key and value rows it reads.  Each of the four
// warps walks its own groups of 8 keys with its own running softmax: a key (or value) row is one
// coalesced warp-wide load (lane t holds dims DPL t .. DPL t + DPL - 1), the 8 key rows and the 8
// value rows of a group are requested together, the 8 x G dot products are reduced with shuffles.
// The warps meet in shared memory; splits of a head are merged in split order by the CTA that
// arrives last.
constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = 4;
constexpr int kKeyGroup = 8;

struct AttnArgs {
  const __nv_bfloat16* q;        // [B, H, Dh], rotated
  const __nv_bfloat16* kcache;   // [rows, S_max, Hk, Dh]
  const __nv_bfloat16* vcache;
  const int* seqlens;
  __nv_bfloat16* out;            // [B, H, Dh]
  float* part;                   // [B, Hk, nsplit, G, Dh + 2] (acc, m, l)
  int* counters;                 // [B, Hk]
  int B, H, Hk, Dh, S_max, nsplit, seqlen_add, shared_cache;
  float scale;
};

template <int DPL>
__device__ __forceinline__ void ld_row(const __nv_bfloat16* row, int lane, float (&f)[DPL]);
template <>
__device__ __forceinline__ void ld_row<4>(const __nv_bfloat16* row, int lane, float (&f)[4]) {
  const uint2 w = __ldg(reinterpret_cast<const uint2*>(row) + lane);
  f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xffff0000u);
  f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xffff0000u);
}
template <>
__device__ __forceinline__ void ld_row<2>(const __nv_bfloat16* row, int lane, float (&f)[2]) {
  const unsigned w = __ldg(reinterpret_cast<const unsigned*>(row) + lane);
  f[0] = __uint_as_float(w << 16); f[1] = __uint_as_float(w & 0xffff0000u);
}

// RB > 1 (prompt pass: the batch rows are consecutive positions of one sequence and share its cache):
// a CTA takes RB consecutive rows of one kv head, so a key / value row is read once for RB x G
// query vectors; every (row, head) slot has its own causal limit.  RB > 1 runs with one split.
template <int DH, int G, int RB>
__global__ void __launch_bounds__(kAttnThreads) batch_attn_kernel(const AttnArgs a) {
  constexpr int DPL = DH / 32;
  constexpr int NG = G * RB;                     // query vectors that share the rows this CTA reads
  __shared__ float wm[kAttnWarps][NG], wl[kAttnWarps][NG];
  __shared__ float wacc[kAttnWarps][NG][DH];
  __shared__ int last_sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  pdl_wait();
  int idx = blockIdx.x;
  const int split = idx % a.nsplit;
  idx /= a.nsplit;
  const int hk = idx % a.Hk, b = idx / a.Hk;     // b: batch row, or block of RB rows
  const int row0 = b * RB;
  int nl[RB];                                    // keys visible to each of the CTA's rows
  int n = 0;
#pragma unroll
  for (int r = 0; r < RB; ++r) {
    const int row = row0 + r;
    nl[r] = row < a.B ? min(a.seqlens[row] + a.seqlen_add, a.S_max) : 0;
    n = max(n, nl[r]);
  }
  const int per = (n + a.nsplit - 1) / a.nsplit;
  const int j0 = min(n, split * per), j1 = min(n, j0 + per);
  const size_t rowstride = (size_t)a.Hk * DH;
  const size_t cbase = ((size_t)(a.shared_cache ? 0 : row0) * a.S_max) * rowstride + (size_t)hk * DH;
  const __nv_bfloat16* kbase = a.kcache + cbase;
  const __nv_bfloat16* vbase = a.vcache + cbase;

  float q[NG][DPL], acc[NG][DPL], m[NG], l[NG];
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int row = min(row0 + g / G, a.B - 1);
    ld_row<DPL>(a.q + ((size_t)row * a.H + hk * G + g % G) * DH, lane, q[g]);
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
      q[g][e] *= a.scale;
      acc[g][e] = 0.0f;
    }
    m[g] = -INFINITY;
    l[g] = 0.0f;
  }

  for (int c0 = j0 + warp * kKeyGroup; c0 < j1; c0 += kAttnWarps * kKeyGroup) {
    const int cn = min(kKeyGroup, j1 - c0);
    float kf[kKeyGroup][DPL], vf[kKeyGroup][DPL];
#pragma unroll
    for (int i = 0; i < kKeyGroup; ++i) {
      const int row = c0 + (i < cn ? i : cn - 1);   // past the end: the last row again, weighted 0 below
      ld_row<DPL>(kbase + (size_t)row * rowstride, lane, kf[i]);
      ld_row<DPL>(vbase + (size_t)row * rowstride, lane, vf[i]);
    }
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      float s[kKeyGroup];
#pragma unroll
      for (int i = 0; i < kKeyGroup; ++i) {
        float d = 0.0f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) d += kf[i][e] * q[g][e];
        s[i] = d;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int i = 0; i < kKeyGroup; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], o);
      }
      float cm = -INFINITY;
#pragma unroll
      for (int i = 0; i < kKeyGroup; ++i) {
        if (i >= cn) s[i] = -INFINITY;                          // past the split
        if (RB > 1 && c0 + i >= nl[g / G]) s[i] = -INFINITY;    // past this query's position
        cm = fmaxf(cm, s[i]);
      }
      const float mn = fmaxf(m[g], cm);
      // (with row blocks a whole group can be invisible to an early row: every weight below is then 0)
      const float mref = (RB > 1 && mn == -INFINITY) ? 0.0f : mn;
      const float corr = __expf(m[g] - mref);               // 0 when m is still -inf
      m[g] = mn;
      float ps = 0.0f;
#pragma unroll
      for (int e = 0; e < DPL; ++e) acc[g][e] *= corr;
#pragma unroll
      for (int i = 0; i < kKeyGroup; ++i) {
        const float pr = __expf(s[i] - mref);               // 0 for the masked rows
        ps += pr;
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[g][e] += pr * vf[i][e];
      }
      l[g] = l[g] * corr + ps;
    }
  }
  // ---- the warps meet
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    if (lane == 0) {
      wm[warp][g] = m[g];
      wl[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < DPL; ++e) wacc[warp][g][lane * DPL + e] = acc[g][e];
  }
  __syncthreads();
  const int nsplit = a.nsplit;
  const int rec = DH + 2;
  float* mine = a.part + ((((size_t)b * a.Hk + hk) * nsplit + split) * NG) * rec;
  for (int i = tid; i < NG * DH; i += kAttnThreads) {
    const int g = i / DH, dd = i - g * DH;
    const int row = row0 + g / G;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, wm[w][g]);
    float num = 0.0f, den = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float wgt = wm[w][g] == -INFINITY ? 0.0f : __expf(wm[w][g] - mm);
      num += wgt * wacc[w][g][dd];
      den += wgt * wl[w][g];
    }
    if (nsplit == 1) {
      if (row < a.B)
        a.out[((size_t)row * a.H + hk * G + g % G) * DH + dd] = __float2bfloat16_rn(den > 0.0f ? num / den : 0.0f);
    } else {
      mine[(size_t)g * rec + dd] = num;
      if (dd == 0) {
        mine[(size_t)g * rec + DH] = mm;
        mine[(size_t)g * rec + DH + 1] = den;
      }
    }
  }
  if (nsplit == 1) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&a.counters[b * a.Hk + hk], 1);
    last_sh = old == nsplit - 1;
    if (old == nsplit - 1) a.counters[b * a.Hk + hk] = 0;
  }
  __syncthreads();
  if (!last_sh) return;
  __threadfence();
  const float* parts = a.part + (((size_t)b * a.Hk + hk) * nsplit) * NG * rec;
  for (int i = tid; i < NG * DH; i += kAttnThreads) {
    const int g = i / DH, dd = i - g * DH;
    const int row = row0 + g / G;
    float mm = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) mm = fmaxf(mm, __ldcg(parts + ((size_t)sp * NG + g) * rec + DH));
    float num = 0.0f, den = 0.0f;
    for (int sp = 0; sp < nsplit; ++sp) {
      const float* pr = parts + ((size_t)sp * NG + g) * rec;
      const float ms = __ldcg(pr + DH);
      const float wgt = ms == -INFINITY ? 0.0f : __expf(ms - mm);
      num += wgt * __ldcg(pr + dd);
      den += wgt * __ldcg(pr + DH + 1);
    }
    if (row < a.B)
      a.out[((size_t)row * a.H + hk * G + g % G) * DH + dd] = __float2bfloat16_rn(den > 0.0f ? num / den : 0.0f);
  }
}

// ------------------------------------------------------------------------------- prompt-pass attention
// Causal attention of a block of consecutive prompt rows over the one sequence's cache, on the
// tensor cores (mma.sync m16n8k16 / bf16, fp32 accumulation): the rows of a pass share the cache
// rows they read, so a key / value block staged in shared memory serves 32 query vectors
// (32 / G rows x G heads of one kv head, 16 per warp).  Per block of 64 keys: S = Q K^T (the key rows
// are the col-major B operand as they lie), causal mask by absolute position, running softmax,
// O += P V with the value fragments taken through ldmatrix.trans.  Replaces the row-block variant
// of batch_attn_kernel for the prompt pass (the reference: kernels/attn/prefill/rope_sdpa.py:67-427).
constexpr int kPfWarps = 2;
constexpr int kPfSlots = 16 * kPfWarps;     // query vectors per CTA
constexpr int kPfKeys = 64;                 // keys per block

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int DH>
__global__ void __launch_bounds__(kPfWarps * 32) prompt_attn_kernel(const AttnArgs a) {
  constexpr int STRIDE = DH * 2 + 16;                 // bytes of a staged row (16 bytes of padding: no bank conflicts)
  constexpr int KS = DH / 16;                         // k-steps of Q K^T
  constexpr int NT = kPfKeys / 8;                     // score tiles per key block
  constexpr int DT = DH / 8;                          // output tiles
  __shared__ __align__(16) unsigned char ks_s[kPfKeys * STRIDE];
  __shared__ __align__(16) unsigned char vs_s[kPfKeys * STRIDE];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  pdl_launch_dependents();
  pdl_wait();
  const int G = a.H / a.Hk;
  const int rpb = kPfSlots / G;                       // rows per CTA
  const int hk = blockIdx.y, row0 = blockIdx.x * rpb;
  // this thread's two query vectors: slots m0 and m0 + 8 of the CTA
  const int m0 = warp * 16 + g;
  int rowq[2], headq[2], nl[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + 8 * i;
    rowq[i] = row0 + m / G;
    headq[i] = hk * G + m % G;
    nl[i] = rowq[i] < a.B ? min(a.seqlens[rowq[i]] + a.seqlen_add, a.S_max) : 0;
  }
  const int last_row = min(row0 + rpb, a.B) - 1;
  const int nmax = last_row >= row0 ? min(a.seqlens[last_row] + a.seqlen_add, a.S_max) : 0;   // positions increase with the row
  // Q fragments (rows g and g + 8 of the warp's 16, dims 16 ks + 2 t .. and + 8)
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const __nv_bfloat16* qp = a.q + ((size_t)min(rowq[i], a.B - 1) * a.H + headq[i]) * DH + ks * 16 + 2 * t;
      qa[ks][i] = *reinterpret_cast<const uint32_t*>(qp);
      qa[ks][2 + i] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.0f, 0.0f};
  const size_t rowstride = (size_t)a.Hk * DH;
  const __nv_bfloat16* kbase = a.kcache + (size_t)hk * DH;     // shared cache: row 0 of the cache tensor
  const __nv_bfloat16* vbase = a.vcache + (size_t)hk * DH;

  for (int k0 = 0; k0 < nmax; k0 += kPfKeys) {
    // ---- stage 64 key rows and 64 value rows (zeros past the visible range)
    __syncthreads();
    for (int i = tid; i < kPfKeys * (DH / 8); i += kPfWarps * 32) {
      const int r = i / (DH / 8), c = i - r * (DH / 8);
      uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
      if (k0 + r < nmax) {
        kv = __ldg(reinterpret_cast<const uint4*>(kbase + (size_t)(k0 + r) * rowstride) + c);
        vv = __ldg(reinterpret_cast<const uint4*>(vbase + (size_t)(k0 + r) * rowstride) + c);
      }
      *reinterpret_cast<uint4*>(ks_s + r * STRIDE + c * 16) = kv;
      *reinterpret_cast<uint4*>(vs_s + r * STRIDE + c * 16) = vv;
    }
    __syncthreads();
    // ---- S = Q K^T for this warp's 16 query vectors x 64 keys
    float sc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f;
      const unsigned char* kr = ks_s + (nt * 8 + g) * STRIDE + 4 * t;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr + ks * 32);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + ks * 32 + 16);
        mma_bf16_16816(sc[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
      }
    }
    // ---- scale, causal mask, running softmax (rows g and g + 8; a row's 64 scores sit in 4 lanes)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int kj = k0 + nt * 8 + 2 * t + (e & 1);
        const float v = kj < nl[i] ? sc[nt][e] * a.scale : -INFINITY;
        sc[nt][e] = v;
        mx[i] = fmaxf(mx[i], v);
      }
    }
    float corr[2], mref[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float mn = fmaxf(mrow[i], mx[i]);
      mref[i] = mn == -INFINITY ? 0.0f : mn;          // nothing visible yet: every weight is 0
      corr[i] = __expf(mrow[i] - mref[i]);
      mrow[i] = mn;
    }
    float ps[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pr = __expf(sc[nt][e] - mref[e >> 1]);
        sc[nt][e] = pr;
        ps[e >> 1] += pr;
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 1);
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 2);
      lrow[i] = lrow[i] * corr[i] + ps[i];
    }
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      o[d][0] *= corr[0]; o[d][1] *= corr[0];
      o[d][2] *= corr[1]; o[d][3] *= corr[1];
    }
    // ---- O += P V: 16 keys per step; the P fragments are the score tiles as they lie
#pragma unroll
    for (int kk = 0; kk < kPfKeys / 16; ++kk) {
      const uint32_t pa0 = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
      const uint32_t pa1 = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
      const uint32_t pa2 = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
      const uint32_t pa3 = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
      // ldmatrix.x4.trans: matrices (keys 16 kk .. + 7, dims 16 j .. + 7), (keys + 8, same dims),
      // (keys .. + 7, dims + 8), (keys + 8, dims + 8) -> b0, b1 of output tile 2 j and of tile 2 j + 1
      const int lrow_ = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const unsigned char* vr = vs_s + lrow_ * STRIDE + ((lane >> 4) & 1) * 16;
#pragma unroll
      for (int j = 0; j < DT / 2; ++j) {
        uint32_t b0, b1, b2, b3;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vr + j * 32);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
        mma_bf16_16816(o[2 * j], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16_16816(o[2 * j + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
    }
  }
  // ---- normalise and store: thread holds (row g, dims 8 d + 2 t, + 1) and (row g + 8, same dims)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (rowq[i] >= a.B) continue;
    const float inv = lrow[i] > 0.0f ? 1.0f / lrow[i] : 0.0f;
    __nv_bfloat16* op = a.out + ((size_t)rowq[i] * a.H + headq[i]) * DH + 2 * t;
#pragma unroll
    for (int d = 0; d < DT; ++d)
      *reinterpret_cast<uint32_t*>(op + d * 8) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
  }
}

// ------------------------------------------------------------------------------- grouped-query decode attention
// Single-query attention for H / Hk = 4 or 8 query heads per kv head on the tensor cores: the G
// heads that share a kv head are the rows of one m16n8k16 tile (rows G .. 15 are zero), so a key /
// value row is read once per sequence and multiplied for all its heads at once, instead of one
// shuffle-reduced dot product per head and key (which ran at 0.9 TB/s for 8 heads per kv head).
// One CTA = (sequence, kv head, key split) as in batch_attn_kernel; each of its 4 warps walks its own blocks of 32 keys: cp.async of the 32 key
// rows and 32 value rows into the warp's own shared-memory stage, S = Q K^T, running softmax,
// O += P V with ldmatrix.trans value fragments (the fragment code of prompt_attn_kernel).  The warps
// merge in shared memory, the splits of a head in split order by the CTA that arrives last.
constexpr int kGqKeys = 32;      // keys per warp block
constexpr int kGqMaxSplit = 64;  // key splits of a sequence at most

template <int DH>
__global__ void __launch_bounds__(kAttnThreads, 3) gqa_decode_attn_kernel(const AttnArgs a) {
  constexpr int STRIDE = DH * 2 + 16;
  constexpr int KS = DH / 16, NT = kGqKeys / 8, DT = DH / 8;
  constexpr int PIECES = DH / 8;                       // 16-byte pieces of a row
  extern __shared__ __align__(16) unsigned char gq_smem[];
  __shared__ int last_sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  pdl_launch_dependents();
  pdl_wait();
  const int G = a.H / a.Hk;
  int idx = blockIdx.x;
  const int split = idx % a.nsplit;
  idx /= a.nsplit;
  const int hk = idx % a.Hk, b = idx / a.Hk;
  const int n = min(a.seqlens[b] + a.seqlen_add, a.S_max);
  const int per = ((n + a.nsplit - 1) / a.nsplit + kGqKeys - 1) / kGqKeys * kGqKeys;   // whole blocks per split
  const int j0 = min(n, split * per), j1 = min(n, j0 + per);
  const size_t rowstride = (size_t)a.Hk * DH;
  const size_t cbase = ((size_t)(a.shared_cache ? 0 : b) * a.S_max) * rowstride + (size_t)hk * DH;
  const __nv_bfloat16* kbase = a.kcache + cbase;
  const __nv_bfloat16* vbase = a.vcache + cbase;
  unsigned char* ks_s = gq_smem + (size_t)warp * (2 * kGqKeys * STRIDE);
  unsigned char* vs_s = ks_s + kGqKeys * STRIDE;

  // Q fragments: row g of the tile = head hk G + g (zero for g >= G), rows 8 .. 15 zero
  uint32_t qa[KS][2];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qa[ks][0] = qa[ks][1] = 0u;
    if (g < G) {
      const __nv_bfloat16* qp = a.q + ((size_t)b * a.H + hk * G + g) * DH + ks * 16 + 2 * t;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  float o[DT][2];
#pragma unroll
  for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = 0.0f;
  float mrow = -INFINITY, lrow = 0.0f;

  for (int k0 = j0 + warp * kGqKeys; k0 < j1; k0 += kAttnWarps * kGqKeys) {
    // ---- stage this warp's 32 key rows and 32 value rows (rows past the split repeat its last row;
    // their scores are masked)
    __syncwarp();
    for (int i = lane; i < kGqKeys * PIECES; i += 32) {
      const int r = i / PIECES, c = i - r * PIECES;
      const size_t src = (size_t)min(k0 + r, j1 - 1) * rowstride + (size_t)c * 8;
      const uint32_t dk = smem_u32(ks_s + r * STRIDE + c * 16), dv = smem_u32(vs_s + r * STRIDE + c * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dk), "l"(kbase + src) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dv), "l"(vbase + src) : "memory");
    }
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    // ---- S = Q K^T: 16 (G used) query heads x 32 keys
    float sc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f;
      const unsigned char* kr = ks_s + (nt * 8 + g) * STRIDE + 4 * t;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr + ks * 32);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + ks * 32 + 16);
        mma_bf16_16816(sc[nt], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
      }
    }
    // ---- scale, mask, running softmax of row g (its 32 scores sit in the 4 lanes of the group)
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kj = k0 + nt * 8 + 2 * t + e;
        const float v = kj < j1 ? sc[nt][e] * a.scale : -INFINITY;
        sc[nt][e] = v;
        mx = fmaxf(mx, v);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(mrow, mx);           // finite: key k0 is inside the split
    const float corr = __expf(mrow - mn);
    mrow = mn;
    float ps = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pr = __expf(sc[nt][e] - mn);
        sc[nt][e] = pr;
        ps += pr;
      }
    }
    ps += __shfl_xor_sync(0xffffffffu, ps, 1);
    ps += __shfl_xor_sync(0xffffffffu, ps, 2);
    lrow = lrow * corr + ps;
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      o[d][0] *= corr;
      o[d][1] *= corr;
    }
    // ---- O += P V, 16 keys per step (rows 8 .. 15 of P are zero)
#pragma unroll
    for (int kk = 0; kk < kGqKeys / 16; ++kk) {
      const uint32_t pa0 = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
      const uint32_t pa2 = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
      const int lr = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const unsigned char* vr = vs_s + lr * STRIDE + ((lane >> 4) & 1) * 16;
#pragma unroll
      for (int j = 0; j < DT / 2; ++j) {
        uint32_t b0, b1, b2, b3;
        const uint32_t addr = (uint32_t)__cvta_generic_to_shared(vr + j * 32);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(addr));
        float c0[4] = {o[2 * j][0], o[2 * j][1], 0.0f, 0.0f}, c1[4] = {o[2 * j + 1][0], o[2 * j + 1][1], 0.0f, 0.0f};
        mma_bf16_16816(c0, pa0, 0u, pa2, 0u, b0, b1);
        mma_bf16_16816(c1, pa0, 0u, pa2, 0u, b2, b3);
        o[2 * j][0] = c0[0]; o[2 * j][1] = c0[1];
        o[2 * j + 1][0] = c1[0]; o[2 * j + 1][1] = c1[1];
      }
    }
  }

  // ---- the four warps meet in shared memory (the stages are free): [warp][head][DH + 4]
  // (DH values, running maximum, running sum; records stay 16-byte aligned)
  constexpr int rec = DH + 4;
  __syncthreads();
  float* wpart = reinterpret_cast<float*>(gq_smem);
  if (g < G) {
    float* mine = wpart + ((size_t)warp * G + g) * rec;
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      mine[d * 8 + 2 * t] = o[d][0];
      mine[d * 8 + 2 * t + 1] = o[d][1];
    }
    if (t == 0) {
      mine[DH] = mrow;
      mine[DH + 1] = lrow;
    }
  }
  __syncthreads();
  const int nsplit = a.nsplit;
  float* gpart = a.part + ((((size_t)b * a.Hk + hk) * nsplit + split) * G) * rec;
  for (int i = tid; i < G * DH; i += kAttnThreads) {
    const int gg = i / DH, dd = i - gg * DH;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, wpart[((size_t)w * G + gg) * rec + DH]);
    float num = 0.0f, den = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* pr = wpart + ((size_t)w * G + gg) * rec;
      const float wgt = pr[DH] == -INFINITY ? 0.0f : __expf(pr[DH] - mm);
      num += wgt * pr[dd];
      den += wgt * pr[DH + 1];
    }
    if (nsplit == 1) {
      a.out[((size_t)b * a.H + hk * G + gg) * DH + dd] = __float2bfloat16_rn(den > 0.0f ? num / den : 0.0f);
    } else {
      gpart[(size_t)gg * rec + dd] = num;
      if (dd == 0) {
        gpart[(size_t)gg * rec + DH] = mm;
        gpart[(size_t)gg * rec + DH + 1] = den;
      }
    }
  }
  if (nsplit == 1) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&a.counters[b * a.Hk + hk], 1);
    last_sh = old == nsplit - 1;
    if (old == nsplit - 1) a.counters[b * a.Hk + hk] = 0;
  }
  __syncthreads();
  if (!last_sh) return;
  __threadfence();
  // ---- merge of the splits by the last CTA: the weight of every (split, head) once, in shared
  // memory, then each thread sums four output dims over the splits with independent 16-byte loads
  const float* parts = a.part + (((size_t)b * a.Hk + hk) * nsplit) * G * rec;
  float* wgt_s = wpart;                          // [nsplit][G] maxima, then weights (<= 64 x 8)
  float* den_s = wpart + kGqMaxSplit * 8;        // [G] sums, [8 + G] maxima
  float* l_s = den_s + 16;                       // [nsplit][G] running sums of the splits
  for (int i = tid; i < nsplit * G; i += kAttnThreads) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(parts + (size_t)i * rec + DH));
    wgt_s[i] = ml.x;
    l_s[i] = ml.y;
  }
  __syncthreads();
  if (tid < G) {
    float mm = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) mm = fmaxf(mm, wgt_s[sp * G + tid]);
    den_s[8 + tid] = mm;
  }
  __syncthreads();
  for (int i = tid; i < nsplit * G; i += kAttnThreads) {
    const float ms = wgt_s[i];
    wgt_s[i] = ms == -INFINITY ? 0.0f : __expf(ms - den_s[8 + i % G]);
  }
  __syncthreads();
  if (tid < G) {
    float den = 0.0f;
    for (int sp = 0; sp < nsplit; ++sp) den += wgt_s[sp * G + tid] * l_s[sp * G + tid];
    den_s[tid] = den;
  }
  __syncthreads();
  for (int i = tid; i < G * (DH / 4); i += kAttnThreads) {
    const int gg = i / (DH / 4), d4 = (i - gg * (DH / 4)) * 4;
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 16
    for (int sp = 0; sp < nsplit; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(parts + ((size_t)sp * G + gg) * rec + d4));
      const float wg = wgt_s[sp * G + gg];
      num.x += wg * v.x; num.y += wg * v.y; num.z += wg * v.z; num.w += wg * v.w;
    }
    const float den = den_s[gg];
    const float inv = den > 0.0f ? 1.0f / den : 0.0f;
    uint2 o2;
    o2.x = pack_bf16(num.x * inv, num.y * inv);
    o2.y = pack_bf16(num.z * inv, num.w * inv);
    *reinterpret_cast<uint2*>(a.out + ((size_t)b * a.H + hk * G + gg) * DH + d4) = o2;
  }
}

// ------------------------------------------------------------------------------- step head / tail
__global__ void embed_rows_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ tokens,
                                  __nv_bfloat16* __restrict__ out, int d, int vocab) {
  const int b = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  int tok = tokens[b];
  tok = min(max(tok, 0), vocab - 1);
  for (int i = threadIdx.x; i < d; i += blockDim.x) out[(size_t)b * d + i] = table[(size_t)tok * d + i];
}

// token[b] = argmax_v logits[b, v] (lowest index among equal maxima); logs it; CTA 0 of the last
// row... every row advances its own sequence length, row 0 the step counter.
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ logits, int vocab, int* tokens,
                                                          int* token_log, int* step_counter, int* seqlens,
                                                          int max_steps, int B) {
  __shared__ float bv[8];
  __shared__ int bi[8];
  const int b = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)b * vocab;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int i = tid; i < vocab; i += 256) {
    const float v = row[i];
    if (v > best || (v == best && i < besti)) {
      best = v;
      besti = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) {
      best = ov;
      besti = oi;
    }
  }
  if ((tid & 31) == 0) {
    bv[tid >> 5] = best;
    bi[tid >> 5] = besti;
  }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < 8; ++i)
      if (bv[i] > best || (bv[i] == best && bi[i] < besti)) {
        best = bv[i];
        besti = bi[i];
      }
    if (besti == 0x7fffffff) besti = 0;
    tokens[b] = besti;
    const int step = *step_counter;
    if (token_log && step < max_steps) token_log[(size_t)step * B + b] = besti;
    seqlens[b] += 1;
  }
}
__global__ void bump_step_kernel(int* step_counter) {
  pdl_launch_dependents();
  pdl_wait();
  *step_counter += 1;
}

// ------------------------------------------------------------------------------- host side
static thread_local char g_err[512];
static int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  fsvd_tile_set_error(code, g_err);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// bf16 [rows, cols] row-major with row stride ld elements, boxes of box_rows x 64 columns, 128-byte swizzle
static int encode_sw128(CUtensorMap* tm, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(FSVD_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16) return fail(FSVD_ERR_ALIGN, "operand rows must start on 16-byte boundaries");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FSVD_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  return 0;
}

static size_t al256(size_t x) { return (x + 255) / 256 * 256; }
static int round16(int b) { return b <= 16 ? 16 : (b + 15) / 16 * 16; }

struct GemmPlan {
  CUtensorMap mapA, mapA2, mapX, mapX2;
  GemmArgs a;
  dim3 grid;
  size_t smem;
};

static int g_sms = 0, g_smem_optin = 0;
static int device_limits() {
  if (g_sms) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(FSVD_ERR_CUDA, "cudaGetDevice failed");
  cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&g_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (g_sms < 1 || g_smem_optin < 64 * 1024) return fail(FSVD_ERR_CUDA, "device limits unavailable");
  return 0;
}

// Segments of the K range: about one CTA per SM, at least 4 k-blocks (64 KB of factor) per CTA
// where the matrix has them, at most kMaxSegs segments, none empty.
static int ctas_per_sm_wanted() {
  static int v = [] {
    const char* e = getenv("FSVD_TILE_CTAS_PER_SM");
    const int x = e ? atoi(e) : 1;
    return x >= 1 && x <= 4 ? x : 1;
  }();
  return v;
}
static void split_k(int tiles, int nkb, int sms, int& segs, int& kbs) {
  int want = (ctas_per_sm_wanted() * sms + tiles / 2) / tiles;
  if (want > kMaxSegs) want = kMaxSegs;
  if (want > nkb / 4) want = nkb / 4;
  if (want < 1) want = 1;
  kbs = (nkb + want - 1) / want;
  segs = (nkb + kbs - 1) / kbs;
}

static unsigned long long* g_tile_trace = nullptr;
static int g_tile_trace_epi = -1;
struct Scratch {
  int* status;
  long long wait_limit;
};

// y[B, P] = epilogue(W[P, K] . x[B, K]^T); W2 / x2: the second accumulator of TE_SWIGLU.
static int plan_gemm(GemmPlan& g, const void* W, const void* W2, int P, int K, int ldw, const void* x, const void* x2,
                     int ldx, int B, int epi, const Scratch& sc, int force_segs = 0) {
  if (int e = device_limits()) return e;
  memset(&g, 0, sizeof(g));
  const int N = round16(B);
  GemmArgs& a = g.a;
  a.P = P; a.K = K; a.B = B; a.N = N;
  a.tiles = (P + kTileM - 1) / kTileM;
  a.nkb = (K + kTileK - 1) / kTileK;
  a.two = W2 ? 1 : 0;
  a.epi = epi;
  const int nacc = a.two ? 2 : 1;
  uint32_t cols = 32;
  while (cols < (uint32_t)(nacc * N)) cols <<= 1;
  a.tmem_cols = cols;
  const size_t stage = (size_t)kWTileBytes * nacc + (size_t)N * 128 * nacc;
  size_t smem = 0;
  int cap = kMaxSegs;
  for (int attempt = 0; attempt < 2; ++attempt) {
    split_k(a.tiles, a.nkb, g_sms, a.segs, a.kbs);
    if (force_segs > 0) {   // the caller wants this many segments (problems of one grouped launch)
      const int want = force_segs < a.nkb ? force_segs : a.nkb;
      a.kbs = (a.nkb + want - 1) / want;
      a.segs = (a.nkb + a.kbs - 1) / a.kbs;
    }
    if (a.segs > cap) {   // second attempt: fewer, longer segments
      a.kbs = (a.nkb + cap - 1) / cap;
      a.segs = (a.nkb + a.kbs - 1) / a.kbs;
    }
    a.cpo = ((N + a.segs - 1) / a.segs + 3) / 4 * 4;   // a multiple of 4: partial sums travel four columns per store
    int ns = (int)((size_t)(g_smem_optin - 2048) / stage);
    if (ns > kMaxStages) ns = kMaxStages;
    if (ns > a.kbs) ns = a.kbs;
    // keep the ring small enough for two CTAs per SM: the clusters of a launch then fit the GPCs in
    // one wave (with one CTA per SM, 24 clusters of 6 do not fit 8 GPCs of 16-20 SMs)
    if (ns > 2 && (size_t)ns * stage > 110 * 1024) {
      ns = (int)((size_t)(110 * 1024) / stage);
      if (ns < 2) ns = 2;
    }
    if (ns < 1) return fail(FSVD_ERR_UNSUPPORTED, "shared memory too small for one stage");
    a.nstages = ns;
    smem = 1024 + (size_t)ns * stage;
    // the ring is reused for the partial sums the cluster's CTAs send each other
    const size_t recv = (size_t)nacc * a.segs * a.cpo * kTileM * 4;
    if (smem < 1024 + recv) smem = 1024 + recv;
    // co-resident CTAs must not ask for more than the 512 tensor-memory columns of an SM
    const size_t floor_smem = (size_t)232448 / (512 / cols + 1) + 1024;
    if (smem < floor_smem) smem = floor_smem;
    // one CTA per SM and more CTAs than SMs would run in two waves: take fewer segments instead
    if (attempt == 0 && smem > 113 * 1024 && a.tiles * a.segs > g_sms && a.segs > 1) {
      cap = g_sms / a.tiles > 0 ? g_sms / a.tiles : 1;
      continue;
    }
    break;
  }
  if (smem > (size_t)g_smem_optin - 1024) return fail(FSVD_ERR_UNSUPPORTED, "shared memory plan exceeds the device limit");
  g.smem = smem;
  g.grid = dim3((unsigned)a.tiles, (unsigned)a.segs);
  a.status = sc.status;
  a.wait_limit = sc.wait_limit;
  a.trace = (g_tile_trace_epi < 0 || g_tile_trace_epi == epi) ? g_tile_trace : nullptr;
  if (int e = encode_sw128(&g.mapA, W, P, K, ldw, kTileM)) return e;
  if (int e = encode_sw128(&g.mapX, x, B, K, ldx, N)) return e;
  if (W2) {
    if (int e = encode_sw128(&g.mapA2, W2, P, K, ldw, kTileM)) return e;
    if (int e = encode_sw128(&g.mapX2, x2, B, K, ldx, N)) return e;
  } else {
    g.mapA2 = g.mapA;
    g.mapX2 = g.mapX;
  }
  return 0;
}

// Launch with the programmatic-stream-serialization attribute (see pdl_wait above).
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, unsigned cluster_y,
                                      cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  if (cluster_y > 0) {
    at[1].id = cudaLaunchAttributeClusterDimension;
    at[1].val.clusterDim.x = 1;
    at[1].val.clusterDim.y = cluster_y;
    at[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  return launch_pdl_cluster(kern, grid, block, smem, 0u, st, std::forward<Args>(args)...);
}

static int launch_group(const GemmPlan* const* plans, int n, cudaStream_t st);
static int launch_gemm(const GemmPlan& g, cudaStream_t st) {
  const GemmPlan* one[1] = {&g};
  return launch_group(one, 1, st);
}
static int launch_group(const GemmPlan* const* plans, int n, cudaStream_t st) {
  static bool attr_set = false;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!attr_set) {
      if (cudaFuncSetAttribute(tile_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g_smem_optin - 1024) != cudaSuccess)
        return fail(FSVD_ERR_CUDA, "cudaFuncSetAttribute failed for the tile kernel");
      attr_set = true;
    }
  }
  GemmGroup grp;
  memset(&grp, 0, sizeof(grp));
  dim3 grid(1, 1, (unsigned)n);
  size_t smem = 0;
  for (int i = 0; i < n; ++i) {
    const GemmPlan& g = *plans[i];
    grp.maps[i][0] = g.mapA; grp.maps[i][1] = g.mapA2; grp.maps[i][2] = g.mapX; grp.maps[i][3] = g.mapX2;
    grp.args[i] = g.a;
    if (g.grid.x > grid.x) grid.x = g.grid.x;
    if (g.grid.y > grid.y) grid.y = g.grid.y;
    if (g.smem > smem) smem = g.smem;
  }
  // grid.y = K segments = CTAs of a cluster (the problems of a group have the same number)
  if (launch_pdl_cluster(tile_gemm_kernel, grid, dim3(kThreads), smem, grid.y, st, grp) != cudaSuccess)
    return fail(FSVD_ERR_CUDA, "tile kernel launch failed");
  fsvd_tile_count_launch();
  return 0;
}

// ---- workspace of the tile path (fsvd_dims with B > 8)
struct TileWs {
  size_t sync, counters, xn, pbuf, qbuf, attn, mid, hact, apart, total;
  int nsplit;
};
static int attn_nsplit(const fsvd_dims& D, int sms) {
  if (D.rows_are_positions) return 1;   // prompt pass: row blocks share the cache rows instead
  if (D.Hk > 0 && D.H / D.Hk >= 4) {
    // grouped-query kernel: 3 CTAs per SM, at least one block of 32 keys for each of a CTA's 4 warps
    int ns = (3 * sms + D.B * D.Hk - 1) / (D.B * D.Hk);
    const int most = (D.S_max + 4 * kGqKeys - 1) / (4 * kGqKeys);
    if (ns > most) ns = most;
    if (ns > kGqMaxSplit) ns = kGqMaxSplit;
    return ns < 1 ? 1 : ns;
  }
  int ns = (8 * sms + D.B * D.Hk - 1) / (D.B * D.Hk);   // about 8 CTAs of 4 warps per SM
  if (ns > 16) ns = 16;
  if (ns < 1) ns = 1;
  return ns;
}
static int imax(int a, int b) { return a > b ? a : b; }
static TileWs tile_layout(const fsvd_dims& D, int sms) {
  TileWs L;
  const int B = D.B;
  const int HD = D.H * D.Dh;
  const int Rqkv = D.Rq + D.Rk + D.Rv;
  size_t o = 0;
  L.sync = o;      o += al256(sizeof(SyncState));
  L.counters = o;  o += al256((size_t)B * D.Hk * 4);   // attention: arrivals of the splits of a head
  L.xn = o;        o += al256((size_t)B * imax(D.d, 8) * 2);
  L.pbuf = o;      o += al256((size_t)B * imax(imax(Rqkv, D.Ru + D.Rg), imax(D.Ro, D.Rd)) * 2);
  L.qbuf = o;      o += al256((size_t)B * HD * 2);
  L.attn = o;      o += al256((size_t)B * HD * 2);
  L.mid = o;       o += al256((size_t)B * D.d * 2);
  L.hact = o;      o += al256((size_t)B * D.I * 2);
  L.nsplit = attn_nsplit(D, sms);
  L.apart = o;     o += al256((size_t)B * D.Hk * L.nsplit * (D.H / imax(D.Hk, 1)) * (D.Dh + 4) * 4);
  L.total = o;
  return L;
}

static int check_tile_dims(const fsvd_dims& D) {
  if (D.dtype != FSVD_DTYPE_BF16) return fail(FSVD_ERR_UNSUPPORTED, "batches above 8 need bf16 factors (dtype 0)");
  if (D.B < 1 || D.B > 128) return fail(FSVD_ERR_UNSUPPORTED, "batch outside 1..128");
  if (D.Dh != 64 && D.Dh != 128) return fail(FSVD_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
  {
    const int G = D.Hk > 0 && D.H % D.Hk == 0 ? D.H / D.Hk : 0;
    if (G != 1 && G != 2 && G != 4 && G != 8) return fail(FSVD_ERR_UNSUPPORTED, "H / Hk must be 1, 2, 4 or 8");
  }
  if (D.Rg != D.Ru) return fail(FSVD_ERR_UNSUPPORTED, "gate and up ranks must be equal for batches above 8");
  const int m8[] = {D.d, D.I, D.Rq, D.Rk, D.Rv, D.Ro, D.Rg, D.Ru, D.Rd};
  for (int v : m8)
    if (v <= 0 || v % 8) return fail(FSVD_ERR_ALIGN, "sizes and ranks must be positive multiples of 8");
  if ((D.H * D.Dh + kTileM - 1) / kTileM > 1024 || (D.Hk * D.Dh + kTileM - 1) / kTileM > 1024)
    return fail(FSVD_ERR_UNSUPPORTED, "more than 1024 row tiles in a q / k / v lift");
  if ((D.d + kTileM - 1) / kTileM > 4096 || (D.I + kTileM - 1) / kTileM > 4096 || (D.vocab + kTileM - 1) / kTileM > 4096)
    return fail(FSVD_ERR_UNSUPPORTED, "more than 4096 row tiles");
  if (D.S_max < 1) return fail(FSVD_ERR_ARG, "S_max");
  return 0;
}

struct LayerPlan {
  GemmPlan g[9];
  AttnArgs at;
};

// The largest segment count, from the largest of the three planned counts (at most the smallest
// number of k-blocks) down to 2, that cuts all three K ranges into exactly that many non-empty
// segments; 0 when there is none.
static int common_segments(int nkb_q, int nkb_k, int nkb_v, int segs_q, int segs_k, int segs_v) {
  auto segs_for = [](int nkb, int want) { const int kbs = (nkb + want - 1) / want; return (nkb + kbs - 1) / kbs; };
  const int nkb_min = std::min(nkb_q, std::min(nkb_k, nkb_v));
  for (int S = std::min(std::max(segs_q, std::max(segs_k, segs_v)), nkb_min); S >= 2; --S)
    if (segs_for(nkb_q, S) == S && segs_for(nkb_k, S) == S && segs_for(nkb_v, S) == S) return S;
  return 0;
}

static int plan_layer(LayerPlan& lp, const fsvd_dims& D, const fsvd_layer& Lw, const void* cos_tab, const void* sin_tab,
                      const int* seqlens, const void* x_in, void* x_out, char* ws, const TileWs& L, long long wait_limit,
                      const void* xn_in = nullptr) {
  const int B = D.B, HD = D.H * D.Dh, KD = D.Hk * D.Dh, Rqkv = D.Rq + D.Rk + D.Rv;
  Scratch sc = {&reinterpret_cast<SyncState*>(ws + L.sync)->status, wait_limit};
  __nv_bfloat16* xn = reinterpret_cast<__nv_bfloat16*>(ws + L.xn);
  __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(ws + L.pbuf);
  __nv_bfloat16* qb = reinterpret_cast<__nv_bfloat16*>(ws + L.qbuf);
  __nv_bfloat16* attn = reinterpret_cast<__nv_bfloat16*>(ws + L.attn);
  __nv_bfloat16* mid = reinterpret_cast<__nv_bfloat16*>(ws + L.mid);
  __nv_bfloat16* hact = reinterpret_cast<__nv_bfloat16*>(ws + L.hact);
  auto rope = [&](GemmArgs& a, void* cache) {
    a.cache = cache; a.cos_tab = cos_tab; a.sin_tab = sin_tab; a.seqlens = seqlens;
    a.Dh = D.Dh; a.HkDh = KD; a.S_max = D.S_max; a.shared_cache = D.rows_are_positions ? 1 : 0;
  };
  int e;
  // 0: [p_q | p_k | p_v] = rms(x) . qkv_v^T
  // xn_in: the caller already holds rms(x) . ln1 (the kernel before this layer wrote it)
  if ((e = plan_gemm(lp.g[0], Lw.qkv_v, nullptr, Rqkv, D.d, D.d, xn_in ? xn_in : xn, nullptr, D.d, B, TE_STORE, sc))) return e;
  lp.g[0].a.out = pb;
  // 1-3: lifts with rotary / cache append
  if ((e = plan_gemm(lp.g[1], Lw.q_u, nullptr, HD, D.Rq, D.Rq, pb, nullptr, Rqkv, B, TE_ROPE_Q, sc))) return e;
  lp.g[1].a.out = qb;
  rope(lp.g[1].a, nullptr);
  if ((e = plan_gemm(lp.g[2], Lw.k_u, nullptr, KD, D.Rk, D.Rk, pb + D.Rq, nullptr, Rqkv, B, TE_ROPE_K, sc))) return e;
  rope(lp.g[2].a, Lw.k_cache);
  if ((e = plan_gemm(lp.g[3], Lw.v_u, nullptr, KD, D.Rv, D.Rv, pb + D.Rq + D.Rk, nullptr, Rqkv, B, TE_VCACHE, sc))) return e;
  rope(lp.g[3].a, Lw.v_cache);
  if (lp.g[1].a.segs != lp.g[2].a.segs || lp.g[1].a.segs != lp.g[3].a.segs) {
    // the three lifts go out as one launch when they cut K into the same number of segments: look for
    // a count (>= 2) that all three can take
    const int S = common_segments(lp.g[1].a.nkb, lp.g[2].a.nkb, lp.g[3].a.nkb, lp.g[1].a.segs, lp.g[2].a.segs, lp.g[3].a.segs);
    if (S >= 2) {
      LayerPlan t = lp;
      const bool planned = !plan_gemm(t.g[1], Lw.q_u, nullptr, HD, D.Rq, D.Rq, pb, nullptr, Rqkv, B, TE_ROPE_Q, sc, S) &&
                           !plan_gemm(t.g[2], Lw.k_u, nullptr, KD, D.Rk, D.Rk, pb + D.Rq, nullptr, Rqkv, B, TE_ROPE_K, sc, S) &&
                           !plan_gemm(t.g[3], Lw.v_u, nullptr, KD, D.Rv, D.Rv, pb + D.Rq + D.Rk, nullptr, Rqkv, B, TE_VCACHE, sc, S);
      // (the shared-memory plan may still have changed a count: then the separate plans stay)
      if (planned && t.g[1].a.segs == S && t.g[2].a.segs == S && t.g[3].a.segs == S) {
        t.g[1].a.out = qb;
        rope(t.g[1].a, nullptr);
        rope(t.g[2].a, Lw.k_cache);
        rope(t.g[3].a, Lw.v_cache);
        for (int i = 1; i < 4; ++i) lp.g[i] = t.g[i];
      }
    }
  }
  // attention
  AttnArgs& at = lp.at;
  memset(&at, 0, sizeof(at));
  at.q = qb; at.kcache = reinterpret_cast<const __nv_bfloat16*>(Lw.k_cache);
  at.vcache = reinterpret_cast<const __nv_bfloat16*>(Lw.v_cache);
  at.seqlens = seqlens; at.out = attn;
  at.part = reinterpret_cast<float*>(ws + L.apart);
  at.counters = reinterpret_cast<int*>(ws + L.counters);
  at.B = B; at.H = D.H; at.Hk = D.Hk; at.Dh = D.Dh; at.S_max = D.S_max; at.nsplit = L.nsplit; at.seqlen_add = 1;
  at.shared_cache = D.rows_are_positions ? 1 : 0;
  at.scale = 1.0f / sqrtf((float)D.Dh);
  // 4-5: o projection + residual
  if ((e = plan_gemm(lp.g[4], Lw.o_v, nullptr, D.Ro, HD, HD, attn, nullptr, HD, B, TE_STORE, sc))) return e;
  lp.g[4].a.out = pb;
  if ((e = plan_gemm(lp.g[5], Lw.o_u, nullptr, D.d, D.Ro, D.Ro, pb, nullptr, D.Ro, B, TE_RESID, sc))) return e;
  lp.g[5].a.out = mid;
  lp.g[5].a.resid = x_in;
  // 6-8: MLP
  if ((e = plan_gemm(lp.g[6], Lw.upgate_v, nullptr, D.Ru + D.Rg, D.d, D.d, xn, nullptr, D.d, B, TE_STORE, sc))) return e;
  lp.g[6].a.out = pb;
  if ((e = plan_gemm(lp.g[7], Lw.gate_u, Lw.up_u, D.I, D.Rg, D.Rg, pb + D.Ru, pb, D.Ru + D.Rg, B, TE_SWIGLU, sc))) return e;
  lp.g[7].a.out = hact;
  if ((e = plan_gemm(lp.g[8], Lw.down_v, nullptr, D.Rd, D.I, D.I, hact, nullptr, D.I, B, TE_STORE, sc))) return e;
  lp.g[8].a.out = pb;
  (void)mid;
  return 0;
}

template <int DH>
static void launch_attn_g(const AttnArgs& at, cudaStream_t st) {
  const unsigned threads = kAttnThreads;
  const int G = at.H / at.Hk;
  if (at.shared_cache && at.nsplit == 1 && at.B >= 16) {
    // prompt pass: tensor-core attention, 32 / G rows of one kv head per CTA
    const int rpb = kPfSlots / G;
    launch_pdl(prompt_attn_kernel<DH>, dim3((unsigned)((at.B + rpb - 1) / rpb), (unsigned)at.Hk), dim3(kPfWarps * 32), 0, st, at);
    return;
  }
  if (at.shared_cache && at.nsplit == 1 && G < 8) {
    // prompt pass: blocks of 8 / G consecutive rows share the key and value rows they read
    const int RB = 8 / G;
    const unsigned grid = (unsigned)(((at.B + RB - 1) / RB) * at.Hk);
    switch (G) {
      case 1: launch_pdl(batch_attn_kernel<DH, 1, 8>, dim3(grid), dim3(threads), 0, st, at); break;
      case 2: launch_pdl(batch_attn_kernel<DH, 2, 4>, dim3(grid), dim3(threads), 0, st, at); break;
      default: launch_pdl(batch_attn_kernel<DH, 4, 2>, dim3(grid), dim3(threads), 0, st, at); break;
    }
    return;
  }
  const unsigned grid = (unsigned)(at.B * at.Hk * at.nsplit);
  switch (G) {
    case 1: launch_pdl(batch_attn_kernel<DH, 1, 1>, dim3(grid), dim3(threads), 0, st, at); break;
    case 2: launch_pdl(batch_attn_kernel<DH, 2, 1>, dim3(grid), dim3(threads), 0, st, at); break;
    default: {
      // 4 or 8 heads per kv head: the heads as rows of a tensor-core tile
      constexpr size_t smem = (size_t)kAttnWarps * 2 * kGqKeys * (DH * 2 + 16);
      static bool attr_set = false;   // per instantiation; set under the planner's lock or at first use
      if (!attr_set) {
        cudaFuncSetAttribute(gqa_decode_attn_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_set = true;
      }
      launch_pdl(gqa_decode_attn_kernel<DH>, dim3(grid), dim3(threads), smem, st, at);
    }
  }
}
static int launch_attn(const AttnArgs& at, cudaStream_t st) {
  if (at.Dh == 128) launch_attn_g<128>(at, st);
  else launch_attn_g<64>(at, st);
  if (cudaGetLastError() != cudaSuccess) return fail(FSVD_ERR_CUDA, "attention kernel launch failed");
  fsvd_tile_count_launch();
  return 0;
}

// The last GEMM of a layer (down lift + residual) is planned per call site: its output buffer
// differs between the per-layer entry point and the model.
static int launch_reduce(const ReduceArgs& r, int rows, cudaStream_t st) {
  // wide rows are cut into four column slices (a cluster of four CTAs per row)
  const unsigned C = (r.d >= 2048 && r.d % 32 == 0) ? 4u : 1u;
  if (launch_pdl_cluster(exchange_reduce_rows_kernel, dim3((unsigned)rows, C), dim3(256), 0, C > 1 ? C : 0u, st, r) != cudaSuccess)
    return fail(FSVD_ERR_CUDA, "exchange kernel launch failed");
  fsvd_tile_count_launch();
  return 0;
}

// r1 / r2 (tensor-parallel layer): the o lift and the down lift push their partial sums to every
// rank; r1 replaces the second RMSNorm (sum + residual + norm), r2 finishes the layer output.
static int run_layer(const LayerPlan& lp, const GemmPlan& down_lift, const fsvd_dims& D, const fsvd_layer& Lw,
                     const void* x_in, char* ws, const TileWs& L, cudaStream_t st, const ReduceArgs* r1 = nullptr,
                     const ReduceArgs* r2 = nullptr, bool have_xn = false) {
  __nv_bfloat16* xn = reinterpret_cast<__nv_bfloat16*>(ws + L.xn);
  const __nv_bfloat16* mid = reinterpret_cast<const __nv_bfloat16*>(ws + L.mid);
  int e;
  if (!have_xn) {
    launch_pdl(rmsnorm_rows_kernel, dim3(D.B), dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16*>(x_in),
               reinterpret_cast<const __nv_bfloat16*>(Lw.ln1_w), xn, D.d, D.eps);
    fsvd_tile_count_launch();
  }
  if ((e = launch_gemm(lp.g[0], st))) return e;
  if (lp.g[1].a.segs == lp.g[2].a.segs && lp.g[1].a.segs == lp.g[3].a.segs) {
    // the q, k and v lifts read the same rank vector and write disjoint outputs: one launch
    // (possible when they cut K into the same number of segments = cluster size)
    const GemmPlan* qkv[3] = {&lp.g[1], &lp.g[2], &lp.g[3]};
    if ((e = launch_group(qkv, 3, st))) return e;
  } else {
    for (int i = 1; i < 4; ++i)
      if ((e = launch_gemm(lp.g[i], st))) return e;
  }
  if ((e = launch_attn(lp.at, st))) return e;
  if ((e = launch_gemm(lp.g[4], st))) return e;
  if ((e = launch_gemm(lp.g[5], st))) return e;
  if (r1) {
    if ((e = launch_reduce(*r1, D.B, st))) return e;
  } else {
    launch_pdl(rmsnorm_rows_kernel, dim3(D.B), dim3(256), 0, st, mid, reinterpret_cast<const __nv_bfloat16*>(Lw.ln2_w), xn,
               D.d, D.eps);
    fsvd_tile_count_launch();
  }
  for (int i = 6; i < 9; ++i)
    if ((e = launch_gemm(lp.g[i], st))) return e;
  if ((e = launch_gemm(down_lift, st))) return e;
  if (r2 && (e = launch_reduce(*r2, D.B, st))) return e;
  if (cudaGetLastError() != cudaSuccess) return fail(FSVD_ERR_CUDA, "kernel launch failed");
  return 0;
}

static int plan_down_lift(GemmPlan& g, const fsvd_dims& D, const fsvd_layer& Lw, void* x_out, char* ws, const TileWs& L,
                          long long wait_limit) {
  Scratch sc = {&reinterpret_cast<SyncState*>(ws + L.sync)->status, wait_limit};
  if (int e = plan_gemm(g, Lw.down_u, nullptr, D.d, D.Rd, D.Rd, ws + L.pbuf, nullptr, D.Rd, D.B, TE_RESID, sc)) return e;
  g.a.out = x_out;
  g.a.resid = ws + L.mid;
  return 0;
}

// Tensor-parallel layer: the plans of the single-GPU layer on the rank's shards, with the two
// residual lifts turned into pushes and the reductions that complete them.
struct TpPlan {
  LayerPlan lp;
  GemmPlan dl;
  ReduceArgs r1, r2;
};
static int plan_tp_layer(TpPlan& tp, const fsvd_dims& D, const fsvd_layer& Lw, const void* cos_tab, const void* sin_tab,
                         const int* seqlens, const void* x_in, const void* xn_in, void* x_out, const void* next_norm_w,
                         void* xn_out, const fsvd_exchange& ex, char* ws, const TileWs& L, long long wait_limit) {
  if (int e = plan_layer(tp.lp, D, Lw, cos_tab, sin_tab, seqlens, x_in, x_out, ws, L, wait_limit, xn_in)) return e;
  if (int e = plan_down_lift(tp.dl, D, Lw, x_out, ws, L, wait_limit)) return e;
  fsvd_exch::Ctrl* ctrl = reinterpret_cast<fsvd_exch::Ctrl*>(ex.geom.region[ex.geom.rank]);
  int* status = &reinterpret_cast<SyncState*>(ws + L.sync)->status;
  auto to_push = [&](GemmPlan& g, ReduceArgs& r, const void* resid, void* out, const void* norm_w, void* xn) -> int {
    if ((unsigned)(g.a.tiles * g.a.segs) > ex.geom.flag_cap) return fail(FSVD_ERR_UNSUPPORTED, "more CTAs in a lift than exchange flags");
    g.a.epi = TE_PUSH;
    g.a.out = nullptr;
    g.a.resid = nullptr;
    g.a.ex = ex.geom;
    g.a.ex_seq = &ctrl->seq;
    memset(&r, 0, sizeof(r));
    r.ex = ex.geom;
    r.ctrl = ctrl;
    r.nflags = g.a.tiles * g.a.segs;
    r.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
    r.out = reinterpret_cast<__nv_bfloat16*>(out);
    r.norm_w = reinterpret_cast<const __nv_bfloat16*>(norm_w);
    r.xn = reinterpret_cast<__nv_bfloat16*>(xn);
    r.d = D.d;
    r.eps = D.eps;
    r.status = status;
    r.wait_limit = wait_limit;
    r.trace = ex.trace_cap ? ex.trace : nullptr;
    r.trace_cap = ex.trace_cap;
    return 0;
  };
  if (int e = to_push(tp.lp.g[5], tp.r1, x_in, ws + L.mid, Lw.ln2_w, ws + L.xn)) return e;
  return to_push(tp.dl, tp.r2, ws + L.mid, x_out, next_norm_w, next_norm_w ? xn_out : nullptr);
}

}  // namespace fsvd_tile

// ------------------------------------------------------------------------------- entry points
using namespace fsvd_tile;

size_t fsvd_tile_workspace_bytes(const fsvd_dims* dims) {
  if (!dims || device_limits()) return 0;
  if (check_tile_dims(*dims)) return 0;
  return tile_layout(*dims, g_sms).total;
}

int fsvd_tile_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab, const void* sin_tab,
                           const int* cache_seqlens, const void* x_in, void* x_out, void* ws, size_t ws_bytes,
                           long long wait_limit, void* stream) {
  const fsvd_dims& D = *dims;
  if (int e = device_limits()) return e;
  if (int e = check_tile_dims(D)) return e;
  const TileWs L = tile_layout(D, g_sms);
  if (!ws || ws_bytes < L.total) return fail(FSVD_ERR_WORKSPACE, "workspace too small for this batch");
  if (x_in == x_out) return fail(FSVD_ERR_ARG, "x_in and x_out must differ");
  // the plans of the last call are kept: a decode loop calls with the same arguments every token
  struct Cached {
    fsvd_dims D;
    fsvd_layer Lw;
    const void *cos_tab, *sin_tab, *x_in;
    const int* seqlens;
    void *x_out, *ws;
    long long wait_limit;
    LayerPlan lp;
    GemmPlan dl;
    bool valid = false;
  };
  static std::mutex mu;
  static std::vector<Cached*> cache;
  std::lock_guard<std::mutex> lock(mu);
  Cached* c = nullptr;
  for (Cached* k : cache)
    if (k->valid && !memcmp(&k->D, &D, sizeof(D)) && !memcmp(&k->Lw, layer, sizeof(*layer)) && k->cos_tab == cos_tab &&
        k->sin_tab == sin_tab && k->x_in == x_in && k->seqlens == cache_seqlens && k->x_out == x_out && k->ws == ws &&
        k->wait_limit == wait_limit)
      c = k;
  if (!c) {
    if (cache.size() >= 128) {
      for (Cached* k : cache) delete k;
      cache.clear();
    }
    c = new Cached();
    c->D = D; c->Lw = *layer; c->cos_tab = cos_tab; c->sin_tab = sin_tab; c->x_in = x_in; c->seqlens = cache_seqlens;
    c->x_out = x_out; c->ws = ws; c->wait_limit = wait_limit;
    int e = plan_layer(c->lp, D, *layer, cos_tab, sin_tab, cache_seqlens, x_in, x_out, reinterpret_cast<char*>(ws), L, wait_limit);
    if (!e) e = plan_down_lift(c->dl, D, *layer, x_out, reinterpret_cast<char*>(ws), L, wait_limit);
    if (e) {
      delete c;
      return e;
    }
    c->valid = true;
    cache.push_back(c);
  }
  return run_layer(c->lp, c->dl, D, *layer, x_in, reinterpret_cast<char*>(ws), L, (cudaStream_t)stream);
}

int fsvd_tile_tp_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab, const void* sin_tab,
                              const int* cache_seqlens, const void* x_in, const void* x_norm_in, void* x_out,
                              const void* next_norm_w, void* x_norm_out, fsvd_exchange* ex, void* ws, size_t ws_bytes,
                              long long wait_limit, void* stream) {
  const fsvd_dims& D = *dims;
  if (int e = device_limits()) return e;
  if (int e = check_tile_dims(D)) return e;
  if (D.rows_are_positions) return fail(FSVD_ERR_UNSUPPORTED, "the tensor-parallel layer takes one row per sequence");
  if (D.d != ex->d || D.B > ex->max_rows) return fail(FSVD_ERR_ARG, "the exchange was created for another width or fewer rows");
  const TileWs L = tile_layout(D, g_sms);
  if (!ws || ws_bytes < L.total) return fail(FSVD_ERR_WORKSPACE, "workspace too small for this batch");
  if (x_in == x_out) return fail(FSVD_ERR_ARG, "x_in and x_out must differ");
  if ((reinterpret_cast<uintptr_t>(x_in) | reinterpret_cast<uintptr_t>(x_out) | reinterpret_cast<uintptr_t>(layer->ln2_w)) & 15)
    return fail(FSVD_ERR_ALIGN, "x_in, x_out and the norm weights must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(x_norm_in) | reinterpret_cast<uintptr_t>(next_norm_w) | reinterpret_cast<uintptr_t>(x_norm_out)) & 15)
    return fail(FSVD_ERR_ALIGN, "x_norm_in, next_norm_w and x_norm_out must be 16-byte aligned");
  if (next_norm_w && !x_norm_out) return fail(FSVD_ERR_ARG, "next_norm_w needs x_norm_out");
  struct Cached {
    fsvd_dims D;
    fsvd_layer Lw;
    const void *cos_tab, *sin_tab, *x_in, *xn_in, *next_w, *xn_out;
    const int* seqlens;
    void *x_out, *ws;
    const fsvd_exchange* ex;
    unsigned long long ex_id;
    long long wait_limit;
    TpPlan tp;
  };
  static std::mutex mu;
  static std::vector<Cached*> cache;
  std::lock_guard<std::mutex> lock(mu);
  Cached* c = nullptr;
  for (Cached* k : cache)
    if (!memcmp(&k->D, &D, sizeof(D)) && !memcmp(&k->Lw, layer, sizeof(*layer)) && k->cos_tab == cos_tab &&
        k->sin_tab == sin_tab && k->x_in == x_in && k->seqlens == cache_seqlens && k->x_out == x_out && k->ws == ws &&
        k->ex == ex && k->ex_id == ex->id && k->wait_limit == wait_limit && k->xn_in == x_norm_in && k->next_w == next_norm_w &&
        k->xn_out == x_norm_out)
      c = k;
  if (!c) {
    if (cache.size() >= 256) {
      for (Cached* k : cache) delete k;
      cache.clear();
    }
    c = new Cached();
    c->D = D; c->Lw = *layer; c->cos_tab = cos_tab; c->sin_tab = sin_tab; c->x_in = x_in; c->seqlens = cache_seqlens;
    c->x_out = x_out; c->ws = ws; c->ex = ex; c->ex_id = ex->id; c->wait_limit = wait_limit;
    c->xn_in = x_norm_in; c->next_w = next_norm_w; c->xn_out = x_norm_out;
    if (int e = plan_tp_layer(c->tp, D, *layer, cos_tab, sin_tab, cache_seqlens, x_in, x_norm_in, x_out, next_norm_w, x_norm_out,
                              *ex, reinterpret_cast<char*>(ws), L, wait_limit)) {
      delete c;
      return e;
    }
    cache.push_back(c);
  }
  return run_layer(c->tp.lp, c->tp.dl, D, *layer, x_in, reinterpret_cast<char*>(ws), L, (cudaStream_t)stream, &c->tp.r1, &c->tp.r2,
                   x_norm_in != nullptr);
}

// ---- whole-model decode for batches above 8: the launches of a step captured once in a CUDA graph
struct fsvd_tile_model {
  fsvd_dims D;
  TileWs L;
  char* ws = nullptr;
  char* extra = nullptr;
  __nv_bfloat16* xbuf[2] = {nullptr, nullptr};
  int *tokens = nullptr, *seqlens = nullptr, *step_counter = nullptr, *token_log = nullptr;
  float* logits = nullptr;
  int max_steps = 0;
  std::vector<LayerPlan> layers;
  std::vector<GemmPlan> down;
  std::vector<fsvd_layer> lw;
  GemmPlan head;
  const void *embed = nullptr, *final_norm = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  long long launches_per_step = 0;
};

static int tile_model_record(fsvd_tile_model* m, cudaStream_t st) {
  const fsvd_dims& D = m->D;
  int e;
  launch_pdl(embed_rows_kernel, dim3(D.B), dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16*>(m->embed),
             (const int*)m->tokens, m->xbuf[0], D.d, D.vocab);
  fsvd_tile_count_launch();
  for (int l = 0; l < D.n_layers; ++l)
    if ((e = run_layer(m->layers[l], m->down[l], D, m->lw[l], m->xbuf[l & 1], m->ws, m->L, st))) return e;
  __nv_bfloat16* xn = reinterpret_cast<__nv_bfloat16*>(m->ws + m->L.xn);
  launch_pdl(rmsnorm_rows_kernel, dim3(D.B), dim3(256), 0, st, (const __nv_bfloat16*)m->xbuf[D.n_layers & 1],
             reinterpret_cast<const __nv_bfloat16*>(m->final_norm), xn, D.d, D.eps);
  fsvd_tile_count_launch();
  if ((e = launch_gemm(m->head, st))) return e;
  launch_pdl(argmax_rows_kernel, dim3(D.B), dim3(256), 0, st, (const float*)m->logits, D.vocab, m->tokens, m->token_log,
             m->step_counter, m->seqlens, m->max_steps, D.B);
  launch_pdl(bump_step_kernel, dim3(1), dim3(1), 0, st, m->step_counter);
  fsvd_tile_count_launch();
  fsvd_tile_count_launch();
  if (cudaGetLastError() != cudaSuccess) return fail(FSVD_ERR_CUDA, "kernel launch failed");
  return 0;
}

int fsvd_tile_model_destroy(fsvd_tile_model* m) {
  if (!m) return 0;
  if (m->exec) cudaGraphExecDestroy(m->exec);
  if (m->graph) cudaGraphDestroy(m->graph);
  cudaFree(m->ws);
  cudaFree(m->extra);
  cudaFree(m->xbuf[0]);
  cudaFree(m->xbuf[1]);
  delete m;
  return 0;
}

int fsvd_tile_model_create(const fsvd_dims* dims, const fsvd_layer* layers, const void* embed, const void* final_norm_w,
                           const void* lm_head, const void* cos_tab, const void* sin_tab, int max_steps, long long wait_limit,
                           fsvd_tile_model** out) {
  const fsvd_dims& D = *dims;
  if (int e = device_limits()) return e;
  if (int e = check_tile_dims(D)) return e;
  if (D.n_layers < 1 || D.vocab < 1) return fail(FSVD_ERR_ARG, "n_layers / vocab");
  if (max_steps < 1) max_steps = 1;
  fsvd_tile_model* m = new fsvd_tile_model();
  m->D = D;
  m->L = tile_layout(D, g_sms);
  m->max_steps = max_steps;
  m->embed = embed;
  m->final_norm = final_norm_w;
  const size_t extra = al256((size_t)D.B * 4) * 2 + al256(4) + al256((size_t)max_steps * D.B * 4) + al256((size_t)D.B * D.vocab * 4);
  cudaError_t ce = cudaMalloc(&m->ws, m->L.total);
  if (ce == cudaSuccess) ce = cudaMalloc(&m->extra, extra);
  if (ce == cudaSuccess) ce = cudaMalloc(&m->xbuf[0], al256((size_t)D.B * D.d * 2));
  if (ce == cudaSuccess) ce = cudaMalloc(&m->xbuf[1], al256((size_t)D.B * D.d * 2));
  if (ce == cudaSuccess) ce = cudaMemset(m->ws, 0, m->L.total);
  if (ce == cudaSuccess) ce = cudaMemset(m->extra, 0, extra);
  if (ce != cudaSuccess) {
    fsvd_tile_model_destroy(m);
    return fail(FSVD_ERR_CUDA, "allocating model scratch failed");
  }
  size_t o = 0;
  m->tokens = reinterpret_cast<int*>(m->extra + o);        o += al256((size_t)D.B * 4);
  m->seqlens = reinterpret_cast<int*>(m->extra + o);       o += al256((size_t)D.B * 4);
  m->step_counter = reinterpret_cast<int*>(m->extra + o);  o += al256(4);
  m->token_log = reinterpret_cast<int*>(m->extra + o);     o += al256((size_t)max_steps * D.B * 4);
  m->logits = reinterpret_cast<float*>(m->extra + o);
  m->layers.resize(D.n_layers);
  m->down.resize(D.n_layers);
  m->lw.assign(layers, layers + D.n_layers);
  int e = 0;
  for (int l = 0; l < D.n_layers && !e; ++l) {
    e = plan_layer(m->layers[l], D, layers[l], cos_tab, sin_tab, m->seqlens, m->xbuf[l & 1], m->xbuf[(l + 1) & 1], m->ws, m->L, wait_limit);
    if (!e) e = plan_down_lift(m->down[l], D, layers[l], m->xbuf[(l + 1) & 1], m->ws, m->L, wait_limit);
  }
  if (!e) {
    Scratch sc = {&reinterpret_cast<SyncState*>(m->ws + m->L.sync)->status, wait_limit};
    e = plan_gemm(m->head, lm_head, nullptr, D.vocab, D.d, D.d, m->ws + m->L.xn, nullptr, D.d, D.B, TE_STORE_F32, sc);
    m->head.a.out = m->logits;
  }
  if (e) {
    fsvd_tile_model_destroy(m);
    return e;
  }
  // capture the launches of one step (nothing runs here; the shared-memory attribute of the GEMM
  // kernel is raised to the device limit first, outside the capture)
  if (cudaFuncSetAttribute(tile_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g_smem_optin - 1024) != cudaSuccess) {
    fsvd_tile_model_destroy(m);
    return fail(FSVD_ERR_CUDA, "cudaFuncSetAttribute failed for the tile kernel");
  }
  cudaStream_t cs = nullptr;
  if (cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking) != cudaSuccess) {
    fsvd_tile_model_destroy(m);
    return fail(FSVD_ERR_CUDA, "cudaStreamCreate failed");
  }
  if (cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal) != cudaSuccess) e = fail(FSVD_ERR_CUDA, "stream capture failed");
  if (!e) {
    const long long before = fsvd_tile_launches();
    e = tile_model_record(m, cs);
    m->launches_per_step = fsvd_tile_launches() - before;
    fsvd_tile_count_launches(-m->launches_per_step);   // recorded, not run
    cudaGraph_t g = nullptr;
    if (cudaStreamEndCapture(cs, &g) != cudaSuccess || !g) e = e ? e : fail(FSVD_ERR_CUDA, "stream capture failed");
    m->graph = g;
  }
  if (!e && cudaGraphInstantiate(&m->exec, m->graph, 0) != cudaSuccess) e = fail(FSVD_ERR_CUDA, "cudaGraphInstantiate failed");
  cudaStreamDestroy(cs);
  if (e) {
    fsvd_tile_model_destroy(m);
    return e;
  }
  *out = m;
  return 0;
}

int fsvd_tile_model_step(fsvd_tile_model* m, int n_steps, void* stream) {
  for (int i = 0; i < n_steps; ++i) {
    if (cudaGraphLaunch(m->exec, (cudaStream_t)stream) != cudaSuccess) return fail(FSVD_ERR_CUDA, "cudaGraphLaunch failed");
    fsvd_tile_count_launches(m->launches_per_step);
  }
  return 0;
}

void fsvd_tile_model_buffers(fsvd_tile_model* m, int** tokens, int** seqlens, int** token_log, int** step_counter,
                             float** logits, float** hidden) {
  if (tokens) *tokens = m->tokens;
  if (seqlens) *seqlens = m->seqlens;
  if (token_log) *token_log = m->token_log;
  if (step_counter) *step_counter = m->step_counter;
  if (logits) *logits = m->logits;
  if (hidden) *hidden = reinterpret_cast<float*>(m->xbuf[m->D.n_layers & 1]);
}
void* fsvd_tile_model_ws(fsvd_tile_model* m) { return m->ws; }
int fsvd_tile_model_launches_per_step(fsvd_tile_model* m) { return (int)m->launches_per_step; }
int fsvd_tile_model_reset(fsvd_tile_model* m, void* stream) {
  if (cudaMemsetAsync(m->ws + m->L.sync, 0, m->L.xn - m->L.sync, (cudaStream_t)stream) != cudaSuccess)
    return fail(FSVD_ERR_CUDA, "cudaMemsetAsync failed");
  return 0;
}

// Debugging aid: while a device buffer is set, every GEMM CTA planned afterwards records nine
// %globaltimer marks (entry, set-up done, dependency met, accumulators done, cluster barrier 1,
// partial sums sent, cluster barrier 2, epilogue done, exit) at [cta][16]; later launches overwrite
// earlier ones.  Not part of the public header.
// Host arithmetic of the planner, callable without a device (unit tests): the K split of a GEMM of
// `tiles` row tiles and `nkb` k-blocks on `sms` SMs, and the segment count the three q / k / v lifts
// can share (0 = none: they go out as separate launches).
extern "C" void fsvd_tile_debug_split_k(int tiles, int nkb, int sms, int* segs, int* kbs) {
  split_k(tiles, nkb, sms, *segs, *kbs);
}
extern "C" int fsvd_tile_debug_common_segments(int nkb_q, int nkb_k, int nkb_v, int segs_q, int segs_k, int segs_v) {
  return common_segments(nkb_q, nkb_k, nkb_v, segs_q, segs_k, segs_v);
}

extern "C" void fsvd_tile_debug_trace(void* dev_ptr) { g_tile_trace = reinterpret_cast<unsigned long long*>(dev_ptr); }
extern "C" void fsvd_tile_debug_trace_epilogue(int epi) { g_tile_trace_epi = epi; }   // -1: every GEMM
