// C ABI of the decode path: builds stage programs on the host and launches the persistent
// interpreter (fsvd_kernel.cuh).  No torch types; see include/flashsvd_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/flashsvd_b200.h"
#include "fsvd_stage.h"
#include "fsvd_tile.h"

using namespace fsvd;


// ------------------------------------------------------------------------------- errors
static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
// hooks for the tiled path (fsvd_tile.cu): same error text, same launch counter
void fsvd_tile_set_error(int, const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }
void fsvd_tile_count_launch() { g_launches.fetch_add(1); }
void fsvd_tile_count_launches(long long n) { g_launches.fetch_add(n); }
long long fsvd_tile_launches() { return g_launches.load(); }
#define CUDA_TRY(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (expr);                                                             \
    if (e_ != cudaSuccess)                                                               \
      return fail(FSVD_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));        \
  } while (0)

// ------------------------------------------------------------------------------- settings
// Process-wide settings of the library (launch geometry, wait budget, trace buffer), guarded by
// one mutex: the entry points may be called from several host threads.
struct Settings {
  int slots = 0, grid = 0;   // ring slots (0 = as many as fit), CTAs (0 = one per SM)
  long long wait_limit = 4000000000ll;   // ~2 s of SM clocks
  unsigned long long* trace = nullptr;
  size_t trace_bytes = 0;
  unsigned generation = 0;   // bumped by every change of the geometry: cached programs of an older one are stale
  int tile_min_batch = 5;    // bf16 batches from this size on take the tiled tensor-core path (FSVD_TILE_MIN_BATCH);
                             // measured crossover on the 7B shape: 4 -> 1315 vs 1211 tokens/s, 5 -> 1282 vs 1465
};
static Settings g_set;
static std::mutex g_set_mu;
static std::once_flag g_set_once;

static int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}
static Settings current_settings() {
  std::call_once(g_set_once, [] {
    g_set.slots = env_int("FSVD_SLOTS", 0);
    g_set.grid = env_int("FSVD_GRID", 0);
    g_set.tile_min_batch = env_int("FSVD_TILE_MIN_BATCH", g_set.tile_min_batch);
    if (g_set.tile_min_batch < 1) g_set.tile_min_batch = 1;
    const char* wl = getenv("FSVD_WAIT_CLOCKS");
    if (wl && *wl && atoll(wl) >= 1000) g_set.wait_limit = atoll(wl);
  });
  std::lock_guard<std::mutex> lock(g_set_mu);
  return g_set;
}

struct DevProps {
  int device = -1, sms = 0, smem_optin = 0;
};
static int get_props(DevProps& p) {
  static DevProps cache[16];
  static std::mutex mu;
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 16 && cache[dev].device == dev) {
    p = cache[dev];
    return 0;
  }
  p.device = dev;
  CUDA_TRY(cudaDeviceGetAttribute(&p.sms, cudaDevAttrMultiProcessorCount, dev));
  CUDA_TRY(cudaDeviceGetAttribute(&p.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  if (dev >= 0 && dev < 16) cache[dev] = p;
  return 0;
}

// Batches that take the tiled tensor-core path (fsvd_tile.cu): always above 8, and bf16 batches from
// the configured size on.
static bool use_tiles(const fsvd_dims& D) {
  return D.B > 8 || (D.dtype == FSVD_DTYPE_BF16 && D.Rg == D.Ru && D.B >= current_settings().tile_min_batch);
}

// ------------------------------------------------------------------------------- kernel table
// The kernel instantiations live in fsvd_inst_*.cu (one translation unit per element type and
// batch width, so they compile in parallel); each exports a table of launchers.
#include "fsvd_launch.h"
extern const KernelEntry g_kernels_bf16[];
extern const KernelEntry g_kernels_f32[];
extern const KernelEntry g_kernels_bf16_q4[];
static const KernelEntry* const g_kernel_tables[] = {g_kernels_bf16, g_kernels_f32, g_kernels_bf16_q4};

// Resolved launch: kernel + geometry for a given dtype / batch.
struct Resolved {
  LaunchFn fn = nullptr;
  int grid = 0, smem_optin = 0, max_slots = 0, device = 0;
  Settings set;
};

static int resolve(int dtype, int B, Resolved& r) {
  r.set = current_settings();
  const Settings& c = r.set;
  DevProps p;
  if (int e = get_props(p)) return e;
  r.device = p.device;
  const int bmax = dtype == FSVD_DTYPE_F32 ? 4 : 8;   // FSVD_DTYPE_BF16_Q4: int4 factors, bf16 everything else
  if (B < 1 || B > bmax) return fail(FSVD_ERR_UNSUPPORTED, "B=%d unsupported (1..%d)", B, bmax);
  r.grid = c.grid > 0 ? (c.grid < p.sms ? c.grid : p.sms) : p.sms;
  r.smem_optin = p.smem_optin;
  r.max_slots = c.slots > 0 ? c.slots : kMaxSlots;
  for (const KernelEntry* tab : g_kernel_tables)
    for (const KernelEntry* kp = tab; kp->fn; ++kp)
      if (kp->dtype == dtype && !r.fn) r.fn = kp->fn;
  if (!r.fn) return fail(FSVD_ERR_UNSUPPORTED, "no kernel for dtype %d", dtype);
  return 0;
}

// ------------------------------------------------------------------------------- TMA descriptors
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
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
static_assert(sizeof(CUtensorMap) == 128, "TMA descriptor size");

// Descriptor of a row-major [rows, cols] matrix with row stride ldw elements, read in boxes of
// kUnitRows rows x kBoxRowBytes bytes; rows and columns outside the matrix read as zeros.
static int encode_map(unsigned char* out, int dtype, const void* base, long long rows, long long cols,
                      long long ldw) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(FSVD_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
  const int esize = dtype == FSVD_DTYPE_BF16 ? 2 : 4;
  if (rows < 1 || cols < 1) return fail(FSVD_ERR_ARG, "empty factor matrix");
  if ((ldw * esize) % 16 || (reinterpret_cast<uintptr_t>(base) & 15))
    return fail(FSVD_ERR_ALIGN, "factor rows must start on 16-byte boundaries");
  CUtensorMap tm;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ldw * esize};
  cuuint32_t box[2] = {(cuuint32_t)(kBoxRowBytes / esize), (cuuint32_t)kUnitRows};
  cuuint32_t es[2] = {1, 1};
  const CUresult r = enc(&tm, dtype == FSVD_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                         2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FSVD_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  memcpy(out, &tm, 128);
  return 0;
}

// Bytes of the int4 tile stream of a [rows, K] factor (fsvd_stage.h describes the tile).
static size_t q4_bytes(long long rows, long long K) {
  const long long rt = (rows + kUnitRows - 1) / kUnitRows, ct = (K + kQ4BoxCols - 1) / kQ4BoxCols;
  return (size_t)(rt * ct) * kQ4BoxBytes;
}
// Descriptor of an int4 tile stream of `tiles` tiles starting at base: a [tiles * 17, 512 bytes]
// matrix of 32-bit words read one tile (17 rows) per box.
static int encode_map_q4(unsigned char* out, const void* base, long long tiles) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(FSVD_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
  if (tiles < 1) return fail(FSVD_ERR_ARG, "empty factor matrix");
  if (reinterpret_cast<uintptr_t>(base) & 15) return fail(FSVD_ERR_ALIGN, "int4 tile streams must start on 16-byte boundaries");
  CUtensorMap tm;
  cuuint64_t dims[2] = {(cuuint64_t)(kQ4RowBytes / 4), (cuuint64_t)tiles * kQ4TileRows};
  cuuint64_t strides[1] = {(cuuint64_t)kQ4RowBytes};
  cuuint32_t box[2] = {(cuuint32_t)(kQ4RowBytes / 4), (cuuint32_t)kQ4TileRows};
  cuuint32_t es[2] = {1, 1};
  const CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FSVD_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  memcpy(out, &tm, 128);
  return 0;
}

// ------------------------------------------------------------------------------- workspace
static size_t al256(size_t x) { return (x + 255) / 256 * 256; }
constexpr int kMaxSegs = 8;
constexpr int kMaxSplit = 32;
constexpr size_t kCounterBytes = 4096;  // B * Hk ints

struct WsLayout {
  size_t sync, pa, pb, hact, qbuf, attn, hidden, part_acc, part_ml, counters, total;
};
static int imax(int a, int b) { return a > b ? a : b; }

static WsLayout ws_layout(const fsvd_dims& D) {
  WsLayout L;
  size_t o = 0;
  const int B = D.B;
  const int maxrank = imax(imax(D.Rq + D.Rk + D.Rv, D.Ru + D.Rg), imax(D.Ro, D.Rd));
  // The barrier words and the attention arrival counters sit at fixed offsets, whatever the
  // shapes: every entry point that shares one workspace finds them where the others left them
  // (zero between launches).
  L.sync = o;      o += al256(sizeof(SyncState));
  L.counters = o;  o += kCounterBytes;
  // pa, pb, hact, attn and hidden hold (fp32, tag) pairs: 8 bytes per element
  L.pa = o;        o += al256((size_t)kMaxSegs * B * maxrank * 8);
  L.pb = o;        o += al256((size_t)kMaxSegs * B * maxrank * 8);
  L.hact = o;      o += al256((size_t)B * imax(D.I, 8) * 8);
  L.qbuf = o;      o += al256((size_t)B * D.H * D.Dh * 4);
  L.attn = o;      o += al256((size_t)B * D.H * D.Dh * 8);
  L.hidden = o;    o += al256((size_t)B * D.d * 8);
  L.part_acc = o;  o += al256((size_t)B * D.H * kMaxSplit * D.Dh * 4);
  L.part_ml = o;   o += al256((size_t)B * D.H * kMaxSplit * 2 * 4);
  L.total = o;
  return L;
}

// ------------------------------------------------------------------------------- builder
struct MapPair {
  unsigned char m[2][128];
};
// What a TMA descriptor of a stage will be made from.  The descriptors are encoded when a program
// is finished and not found among the cached ones: a per-op call that repeats an earlier call
// (same pointers and sizes) then costs no driver call.
struct MapReq {
  int kind = 0;   // 0 none, 1 dense [rows, cols] with row stride ldw, 2 int4 tile stream of `rows` tiles
  const void* base = nullptr;
  long long rows = 0, cols = 0, ldw = 0;
};

struct Builder {
  std::vector<Stage> st;
  std::vector<MapPair> maps;   // TMA descriptors of st[i] (zeros for stages without factors)
  std::vector<MapReq> reqs;    // two per stage: what maps[i].m[0] / m[1] are encoded from
  int grid, TW, B, esize, dtype, boxcols, max_slots;
  long long cum_units = 0;   // GEMV units handed out so far (rotates the unit -> CTA map)
  long long cum_items = 0;   // attention items handed out so far (item -> warp map)
  int max_vec = 8;           // elements of the staged vector a lane may touch, per batch row
  int err = 0;               // first error of gemv()
  bool wq4 = false;          // factors are int4 tile streams (FSVD_DTYPE_BF16_Q4)

  Builder(const Resolved& r, int dtype_, int B_) {
    grid = r.grid;
    TW = r.grid * kConsumerWarps;
    wq4 = dtype_ == FSVD_DTYPE_BF16_Q4;
    dtype = wq4 ? FSVD_DTYPE_BF16 : dtype_;
    esize = dtype == FSVD_DTYPE_BF16 ? 2 : 4;
    boxcols = kBoxRowBytes / esize;
    B = B_;
    max_slots = r.max_slots;
  }
  Stage blank() {
    Stage s;
    memset(&s, 0, sizeof(s));
    s.B = B;
    s.segs = 1;
    s.cps = 1;
    return s;
  }
  void push(const Stage& s) {
    st.push_back(s);
    MapPair z;
    memset(&z, 0, sizeof(z));
    maps.push_back(z);
    reqs.push_back(MapReq());
    reqs.push_back(MapReq());
  }
  void request(int which, int kind, const void* base, long long rows, long long cols, long long ldw) {
    MapReq& q = reqs[2 * (st.size() - 1) + which];
    q.kind = kind; q.base = base; q.rows = rows; q.cols = cols; q.ldw = ldw;
  }
  // ST_ATTN: CTAs per head group (a head group = 1 query head, or 2 that share a kv head) and
  // the rotation of the slice -> CTA map.  Every CTA cuts its part of the keys into 7 splits, one
  // per consumer warp.
  bool has_attn = false;
  int attn_rec_floats = 0;
  void attn_geometry(Stage& s) {
    const int G = s.H / s.Hk, GI = (G % 2 == 0) ? 2 : 1;
    const long long groups = (long long)s.B * s.H / GI;
    int cph = (int)(grid / (groups > 0 ? groups : 1));
    if (cph < 1) cph = 1;
    if (cph > kMaxSplit / kConsumerWarps) cph = kMaxSplit / kConsumerWarps;
    s.nsplit = cph * kConsumerWarps;
    s.rot = (int)(cum_items % grid);
    cum_items += groups * cph;
    has_attn = true;
    // partial results of the warps + per-warp score tiles [rows][33] and probabilities [rows]
    // (rows = query heads of the group x cache rows per chunk: 10 for one head, 2 x 12 for two)
    const int rows = GI == 1 ? 10 : 24;
    const int need = kConsumerWarps * GI * (s.Dh + 2) + kConsumerWarps * rows * 34;
    if (need > attn_rec_floats) attn_rec_floats = need;
  }
  // GEMV stage.  Units (16 rows x one K segment) go round-robin to the CTAs; with split_k the K
  // range is cut into the number of segments (<= kMaxSegs) that gives the busiest CTA the fewest
  // boxes.  rows_total: rows of the matrices behind WA (and WB) that the descriptors may read.
  // Pointer to row `rows` (a multiple of 16 for int4) of a [*, K] factor that starts at base.
  const void* row_ptr(const void* base, long long rows, int K) const {
    const size_t off = wq4 ? q4_bytes(rows, K) : (size_t)rows * K * esize;
    return reinterpret_cast<const char*>(base) + off;
  }
  // seg_x: the input is a T vector copied as it is (VL_SUM with SF_IN_T); when it is longer than
  // 4 KB the K segments are restricted to divisors of the grid so that every CTA works in one
  // segment and stages only that part of the input (SF_SEG_X): a shorter stage-in, and with several
  // batch rows the staged vector no longer takes the shared memory the ring needs.
  Stage& gemv(const void* WA, const void* WB, int P, int K, int ldw, bool split_k, int rope_half = 0,
              int q4_override = -1, bool seg_x = false) {
    const bool q4 = q4_override < 0 ? wq4 : q4_override != 0;
    const int boxcols = q4 ? kQ4BoxCols : this->boxcols;
    const int boxbytes = q4 ? kQ4BoxBytes : kBoxBytes;
    Stage s = blank();
    if (q4) s.flags |= SF_Q4;
    s.type = ST_GEMV;
    s.WA = WA;
    s.WB = WB;
    s.P = P;
    s.K = K;
    s.ldw = ldw;
    s.rope_half = rope_half;
    const int groups = (P + kUnitRows - 1) / kUnitRows;
    const int nchunks = (K + boxcols - 1) / boxcols;
    int best_segs = 1, best_cps = nchunks;
    const bool local = seg_x && split_k && (long long)K * esize > 4096;
    if (split_k) {
      long long best_cost = -1;
      for (int segs = local ? 2 : 1; segs <= kMaxSegs && segs <= nchunks; ++segs) {
        const int cps = (nchunks + segs - 1) / segs;
        const int real = (nchunks + cps - 1) / cps;
        if (real != segs) continue;
        if (local && grid % segs) continue;
        const long long units = (long long)groups * real;
        // time of the busiest CTA's boxes at an SM's share of HBM bandwidth (44 bytes/ns), plus
        // the time every CTA of the next stage spends reading `real` partial vectors from L2
        // (4 bytes/ps over the whole GPU)
        const long long cost = ((units + grid - 1) / grid) * cps * (boxbytes / 44) +
                               (long long)real * P * 4 * grid / 4000;
        if (best_cost < 0 || cost < best_cost) {
          best_cost = cost;
          best_segs = real;
          best_cps = cps;
        }
      }
    }
    s.segs = best_segs;
    s.cps = best_cps;
    if (local && best_segs > 1 && grid % best_segs == 0) s.flags |= SF_SEG_X;
    s.kseg = best_cps * boxcols;
    s.nch = q4 ? nchunks : 0;
    s.rot = (int)(cum_units % grid);
    cum_units += (long long)groups * best_segs;
    push(s);
    // rows behind the pointers: a rotary stage reads physical rows [0, 2P) through WA and
    // [half, 2P) through WB = WA + half rows
    const long long rowsA = rope_half > 0 ? 2ll * P : P;
    const long long rowsB = rope_half > 0 ? 2ll * P - rope_half : P;
    if (rope_half > 0 && rope_half % kUnitRows && !err)
      err = fail(FSVD_ERR_UNSUPPORTED, "head_dim/2 = %d must be a multiple of %d", rope_half, kUnitRows);
    if (q4) {
      // tile rows behind the pointers (a rotary stage's second operand starts rope_half rows in)
      const long long trA = (rowsA + kUnitRows - 1) / kUnitRows;
      const long long trB = rope_half > 0 ? trA - rope_half / kUnitRows : trA;
      request(0, 2, WA, trA * nchunks, 0, 0);
      if (WB) request(1, 2, WB, trB * nchunks, 0, 0);
    } else {
      request(0, 1, WA, rowsA, K, ldw);
      if (WB) request(1, 1, WB, rowsB, K, ldw);
    }
    return st.back();
  }
  // Input vector of the stage just appended (s must be st.back()).  `barrier`: the vector is
  // produced by earlier stages of this program, so the stage waits at a grid barrier and the
  // stage before it arrives there.
  void vec(Stage& s, int mode, const void* src, int len, int nseg, bool barrier) {
    s.vl_mode = mode;
    s.vl_src = src;
    s.vl_len = len;
    s.vl_nseg = nseg;
    if (barrier) need_barrier(s);
    const int staged = (s.flags & SF_SEG_X) ? (len < s.kseg ? len : s.kseg) : len;
    if (staged > max_vec) max_vec = staged;
  }
  void need_barrier(Stage& s) {
    s.flags |= SF_BARRIER;
    if (st.size() >= 2) st[st.size() - 2].flags |= SF_ARRIVE;
  }
  int last() const { return (int)st.size() - 1; }

  // Shared memory the program needs beyond the header and the ring: warps' partial sums and the
  // staged vector.
  int part_bytes() const {
    long long mx = 0;
    for (const Stage& s : st) {
      if (s.type != ST_GEMV) continue;
      const long long units = (long long)((s.P + kUnitRows - 1) / kUnitRows) * s.segs;
      const long long nu = (units + grid - 1) / grid;
      const long long kk = s.cps < kConsumerWarps ? s.cps : kConsumerWarps;
      const long long b = nu * (s.WB ? 2 : 1) * kk * kUnitRows * B * 4;
      if (b > mx) mx = b;
    }
    if (has_attn && (long long)attn_rec_floats * 4 > mx) mx = (long long)attn_rec_floats * 4;
    return (int)((mx + 255) / 256 * 256);
  }
  // Row stride of the staged vector: the longest vector, or the furthest column a box of a K
  // segment can reach (boxes run past K in whole boxes and read zeros from the factor side).
  int xstride() const {
    long long mx = max_vec;
    for (const Stage& s : st) {
      if (s.type != ST_GEMV) continue;
      // (the fused q/k/v lift reads the inputs of its three parts at 0, K and 2 K)
      const long long reach = (long long)(s.xA_off > s.xB_off ? s.xA_off : s.xB_off) +
                              (s.epi == EPI_QKV ? 2ll * s.K : 0ll) +
                              (long long)((s.flags & SF_SEG_X) ? 1 : s.segs) * s.cps *
                                  ((s.flags & SF_Q4) ? kQ4BoxCols : boxcols);
      if (reach > mx) mx = reach;
    }
    return (int)((mx + 7) / 8 * 8) + 8;   // + 16 bytes so that batch rows start in different banks
  }
  int vec_bytes() const { return (B * xstride() * esize + 15) / 16 * 16; }
  // Ring slots: as many as fit beside the rest; a multiple of the consumer warps, or fewer than
  // that when a huge input vector leaves less room (then one warp per slot works).
  int slot_bytes() const {
    for (const Stage& s : st)
      if (s.type == ST_GEMV && (s.flags & SF_Q4)) return kQ4BoxBytes;
    return kBoxBytes;
  }
  int nslots(int smem_optin) const {
    const long long rest = (long long)smem_optin - smem_header_bytes() - part_bytes() - vec_bytes();
    long long n = rest / slot_bytes();
    if (n > max_slots) n = max_slots;
    if (n > kMaxSlots) n = kMaxSlots;
    if (n >= kConsumerWarps) n = n / kConsumerWarps * kConsumerWarps;
    return n < 0 ? 0 : (int)n;
  }
  size_t smem_bytes(int slots) const {
    return (size_t)smem_header_bytes() + (size_t)slots * slot_bytes() + part_bytes() + vec_bytes();
  }
};

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_dims(const fsvd_dims& D) {
  if (D.dtype != FSVD_DTYPE_BF16 && D.dtype != FSVD_DTYPE_F32 && D.dtype != FSVD_DTYPE_BF16_Q4)
    return fail(FSVD_ERR_ARG, "bad dtype %d", D.dtype);
  const int bmax = D.dtype == FSVD_DTYPE_F32 ? 4 : 8;
  if (D.B < 1 || D.B > bmax) return fail(FSVD_ERR_UNSUPPORTED, "B=%d unsupported (1..%d)", D.B, bmax);
  if ((size_t)D.B * D.Hk * sizeof(int) > kCounterBytes)
    return fail(FSVD_ERR_UNSUPPORTED, "B * Hk = %d exceeds the attention counters (%d)", D.B * D.Hk,
                (int)(kCounterBytes / sizeof(int)));
  // the kernel's index arithmetic divides through fp32 reciprocals, exact below 2^22
  const int big[] = {D.d, D.I, D.S_max, D.vocab, D.H * D.Dh};
  for (int v : big)
    if (v >= (1 << 21)) return fail(FSVD_ERR_UNSUPPORTED, "dimension %d is beyond the supported 2^21", v);
  if (D.Dh != 64 && D.Dh != 128) return fail(FSVD_ERR_UNSUPPORTED, "head_dim %d unsupported (64, 128)", D.Dh);
  if (D.Hk < 1 || D.H % D.Hk) return fail(FSVD_ERR_ARG, "H=%d not a multiple of Hk=%d", D.H, D.Hk);
  const int G = D.H / D.Hk;
  if (G != 1 && G != 2 && G != 4 && G != 8) return fail(FSVD_ERR_UNSUPPORTED, "H/Hk=%d unsupported (1,2,4,8)", G);
  const int m8[] = {D.d, D.I, D.Rq, D.Rk, D.Rv, D.Ro, D.Rg, D.Ru, D.Rd};
  for (int v : m8)
    if (v <= 0 || v % 8) return fail(FSVD_ERR_ALIGN, "sizes and ranks must be positive multiples of 8 (got %d)", v);
  if (D.S_max < 1) return fail(FSVD_ERR_ARG, "S_max=%d", D.S_max);
  if ((size_t)D.B * D.H * 4 > kCounterBytes) return fail(FSVD_ERR_UNSUPPORTED, "B*H=%d too large", D.B * D.H);
  return 0;
}

// True when q_u, k_u and v_u lie back to back in memory with one rank: they then form one
// [(H + 2 Hk) * Dh, R] matrix and the three lifts run as one stage (packing.pack_layer and
// synthetic.random_packed_layers lay them out like this).
static bool qkv_lifts_packed(const Builder& b, const void* q_u, const void* k_u, const void* v_u, int H, int Hk,
                             int Dh, int Rq, int Rk, int Rv) {
  if (Rq != Rk || Rq != Rv) return false;
  return k_u == b.row_ptr(q_u, (long long)H * Dh, Rq) && v_u == b.row_ptr(k_u, (long long)Hk * Dh, Rq);
}

struct LayerIO {
  const void* x_in;    // hidden state [B, d] of type T read by the first RMSNorm and residual
  bool x_in_barrier;   // x_in is written by the preceding stage of the same program
  void* x_out;         // hidden state [B, d] of type T written by the last residual
  const int* seqlens;
  const void* cos_tab;
  const void* sin_tab;
};

// Appends the stages of one decoder layer.  Rank-space partial sums travel as fp32, every other
// activation (attention output, SwiGLU activation, hidden state) as T, which is where the
// PyTorch path rounds them.
static void build_layer(Builder& b, const fsvd_dims& D, const fsvd_layer& Lw, const LayerIO& io,
                        char* ws, const WsLayout& L) {
  const size_t first_stage = b.st.size();
  void* pa = ws + L.pa;
  void* pb = ws + L.pb;
  void* hact = ws + L.hact;
  float* qbuf = reinterpret_cast<float*>(ws + L.qbuf);
  void* attn = ws + L.attn;
  void* mid = ws + L.hidden;
  const int Rqkv = D.Rq + D.Rk + D.Rv, HD = D.H * D.Dh, half = D.Dh / 2;

  {  // 1. rank projection of q/k/v on the normalised hidden state
    Stage& s = b.gemv(Lw.qkv_v, nullptr, Rqkv, D.d, D.d, true);
    b.vec(s, VL_RMSNORM, io.x_in, D.d, 1, io.x_in_barrier);
    s.flags |= SF_IN_T;
    s.vl_w = Lw.ln1_w;
    s.eps = D.eps;
    s.epi = EPI_PARTIAL;
    s.out = pa;
  }
  const int segs1 = b.st.back().segs;
  if (qkv_lifts_packed(b, Lw.q_u, Lw.k_u, Lw.v_u, D.H, D.Hk, D.Dh, D.Rq, D.Rk, D.Rv)) {
    // 2-4. q, k and v lifts as one stage over the packed [q_u; k_u; v_u] matrix
    Stage& s = b.gemv(Lw.q_u, b.row_ptr(Lw.q_u, half, D.Rq),
                      (D.H + 2 * D.Hk) * half, D.Rq, D.Rq, false, half);
    b.vec(s, VL_SUM, pa, Rqkv, segs1, true);
    s.rope_half = half;
    s.xA_off = s.xB_off = 0;
    s.epi = EPI_QKV;
    s.out = qbuf;
    s.cache = Lw.k_cache;
    s.vcache = Lw.v_cache;
    s.cos_tab = io.cos_tab; s.sin_tab = io.sin_tab; s.seqlens = io.seqlens;
    s.H = D.H; s.Hk = D.Hk; s.Dh = D.Dh; s.S_max = D.S_max;
  } else {
    {  // 2. lift q with rotary
      Stage& s = b.gemv(Lw.q_u, b.row_ptr(Lw.q_u, half, D.Rq),
                        D.H * half, D.Rq, D.Rq, false, half);
      b.vec(s, VL_SUM, pa, Rqkv, segs1, true);
      s.rope_half = half;
      s.xA_off = s.xB_off = 0;
      s.epi = EPI_ROPE_Q;
      s.out = qbuf;
      s.cos_tab = io.cos_tab; s.sin_tab = io.sin_tab; s.seqlens = io.seqlens;
      s.H = D.H; s.Hk = D.Hk; s.Dh = D.Dh; s.S_max = D.S_max;
    }
    {  // 3. lift k with rotary into the cache
      Stage& s = b.gemv(Lw.k_u, b.row_ptr(Lw.k_u, half, D.Rk),
                        D.Hk * half, D.Rk, D.Rk, false, half);
      s.rope_half = half;
      s.xA_off = s.xB_off = D.Rq;
      s.epi = EPI_ROPE_K;
      s.cache = Lw.k_cache;
      s.cos_tab = io.cos_tab; s.sin_tab = io.sin_tab; s.seqlens = io.seqlens;
      s.H = D.H; s.Hk = D.Hk; s.Dh = D.Dh; s.S_max = D.S_max;
    }
    {  // 4. lift v into the cache
      Stage& s = b.gemv(Lw.v_u, nullptr, D.Hk * D.Dh, D.Rv, D.Rv, false);
      s.xA_off = D.Rq + D.Rk;
      s.epi = EPI_V;
      s.cache = Lw.v_cache;
      s.seqlens = io.seqlens;
      s.H = D.H; s.Hk = D.Hk; s.Dh = D.Dh; s.S_max = D.S_max;
    }
  }
  {  // 5. attention over the cache including the token just appended
    Stage s = b.blank();
    s.type = ST_ATTN;
    s.flags = SF_OUT_T;
    s.q = qbuf;
    s.kcache = Lw.k_cache;
    s.vcache = Lw.v_cache;
    s.seqlens = io.seqlens;
    s.seqlen_add = 1;
    s.out = attn;
    s.part_acc = reinterpret_cast<float*>(ws + L.part_acc);
    s.part_ml = reinterpret_cast<float*>(ws + L.part_ml);
    s.counters = reinterpret_cast<int*>(ws + L.counters);
    s.H = D.H; s.Hk = D.Hk; s.Dh = D.Dh; s.S_max = D.S_max;
    s.scale = 1.0f / sqrtf((float)D.Dh);
    b.attn_geometry(s);
    b.push(s);
    b.need_barrier(b.st.back());
  }
  {  // 6. o rank projection
    Stage& s = b.gemv(Lw.o_v, nullptr, D.Ro, HD, HD, true, 0, -1, true);
    b.vec(s, VL_SUM, attn, HD, 1, true);
    s.flags |= SF_IN_T;
    s.epi = EPI_PARTIAL;
    s.out = pb;
  }
  const int segs6 = b.st.back().segs;
  {  // 7. o lift + residual
    Stage& s = b.gemv(Lw.o_u, nullptr, D.d, D.Ro, D.Ro, false);
    b.vec(s, VL_SUM, pb, D.Ro, segs6, true);
    s.epi = EPI_RESID;
    s.resid = io.x_in;
    s.flags |= SF_RESID_T | SF_OUT_T;
    s.out = mid;
  }
  {  // 8. MLP rank projection on the normalised hidden state: [p_up | p_gate]
    Stage& s = b.gemv(Lw.upgate_v, nullptr, D.Ru + D.Rg, D.d, D.d, true);
    b.vec(s, VL_RMSNORM, mid, D.d, 1, true);
    s.flags |= SF_IN_T;
    s.vl_w = Lw.ln2_w;
    s.eps = D.eps;
    s.epi = EPI_PARTIAL;
    s.out = pa;
  }
  const int segs8 = b.st.back().segs;
  {  // 9. gate/up lift + SiLU·mul
    Stage& s = b.gemv(Lw.gate_u, Lw.up_u, D.I, D.Rg, D.Rg, false);
    b.vec(s, VL_SUM, pa, D.Ru + D.Rg, segs8, true);
    s.xA_off = D.Ru;  // gate input follows the up input
    s.xB_off = 0;
    s.epi = EPI_SWIGLU;
    s.flags |= SF_OUT_T;
    s.out = hact;
  }
  {  // 10. down rank projection
    Stage& s = b.gemv(Lw.down_v, nullptr, D.Rd, D.I, D.I, true, 0, -1, true);
    b.vec(s, VL_SUM, hact, D.I, 1, true);
    s.flags |= SF_IN_T;
    s.epi = EPI_PARTIAL;
    s.out = pb;
  }
  const int segs10 = b.st.back().segs;
  {  // 11. down lift + residual
    Stage& s = b.gemv(Lw.down_u, nullptr, D.d, D.Rd, D.Rd, false);
    b.vec(s, VL_SUM, pb, D.Rd, segs10, true);
    s.epi = EPI_RESID;
    s.resid = mid;
    s.flags |= SF_RESID_T | SF_OUT_T;
    s.out = io.x_out;
  }
  // a chunk of one sequence's prompt: every row uses cache row 0
  if (D.rows_are_positions)
    for (size_t i = first_stage; i < b.st.size(); ++i)
      if (b.st[i].cache || b.st[i].kcache) b.st[i].flags |= SF_SHARED_CACHE;
}

static int check_layer_ptrs(const fsvd_layer& Lw) {
  const void* ps[] = {Lw.ln1_w, Lw.qkv_v, Lw.q_u, Lw.k_u, Lw.v_u, Lw.o_v, Lw.o_u, Lw.ln2_w,
                      Lw.upgate_v, Lw.gate_u, Lw.up_u, Lw.down_v, Lw.down_u, Lw.k_cache, Lw.v_cache};
  for (const void* p : ps) {
    if (!p) return fail(FSVD_ERR_ARG, "null layer pointer");
    if (!aligned16(p)) return fail(FSVD_ERR_ALIGN, "layer pointer %p is not 16-byte aligned", p);
  }
  return 0;
}

// Shared-memory plan of a finished program: ring slots and total bytes.
static int plan_smem(const Resolved& r, const Builder& b, int& slots, size_t& smem) {
  if (b.err) return b.err;
  slots = b.nslots(r.smem_optin);
  if (slots < 1)
    return fail(FSVD_ERR_UNSUPPORTED,
                "shared memory: %d bytes of partial sums and %d bytes of input vector leave no room for the ring (%d available)",
                b.part_bytes(), b.vec_bytes(), r.smem_optin);
  smem = b.smem_bytes(slots);
  return 0;
}

// ------------------------------------------------------------------------------- per-op launches
// Encodes the TMA descriptors a finished program asked for.
static int encode_all(Builder& b) {
  for (size_t i = 0; i < b.reqs.size(); ++i) {
    const MapReq& q = b.reqs[i];
    unsigned char* out = b.maps[i / 2].m[i & 1];
    int e = 0;
    if (q.kind == 1) e = encode_map(out, b.dtype, q.base, q.rows, q.cols, q.ldw);
    else if (q.kind == 2) e = encode_map_q4(out, q.base, q.rows);
    if (e) return e;
  }
  return 0;
}

// A by-value program ready to launch.  The per-op entry points keep the programs they launched in
// a small cache keyed by the program itself (its stage list holds every pointer and size of the
// call), the device and the launch settings, so that a decode loop that calls the same op with
// the same buffers every token plans its shared memory and encodes its TMA descriptors once.
struct SmallLaunch {
  std::vector<Stage> key;   // the stage list the entry was built from
  int device = -1;
  unsigned generation = 0;
  SyncState* sync = nullptr;
  SmallProgram sp;
  SmallMaps sm;
  LaunchArgs a;
  LaunchFn fn = nullptr;
};
constexpr int kLaunchCache = 64;
static SmallLaunch* g_cache[kLaunchCache] = {nullptr};
static int g_cache_next = 0;
static std::mutex g_cache_mu;

static bool same_program(const SmallLaunch& c, const Resolved& r, const Builder& b, SyncState* sync) {
  return c.device == r.device && c.generation == r.set.generation && c.sync == sync && c.fn == r.fn &&
         c.key.size() == b.st.size() && memcmp(c.key.data(), b.st.data(), sizeof(Stage) * b.st.size()) == 0;
}

static int launch_small(const Resolved& r, Builder& b, SyncState* sync, cudaStream_t stream) {
  if ((int)b.st.size() > kMaxSmallStages) return fail(FSVD_ERR_UNSUPPORTED, "program too long");
  if (b.err) return b.err;
  std::lock_guard<std::mutex> lock(g_cache_mu);
  SmallLaunch* sl = nullptr;
  for (SmallLaunch* c : g_cache)
    if (c && same_program(*c, r, b, sync)) sl = c;
  if (!sl) {
    int slots = 0;
    size_t smem = 0;
    if (int e = plan_smem(r, b, slots, smem)) return e;
    if (int e = encode_all(b)) return e;
    sl = new SmallLaunch();
    sl->key = b.st;
    sl->device = r.device;
    sl->generation = r.set.generation;
    sl->sync = sync;
    sl->fn = r.fn;
    memset(&sl->sp, 0, sizeof(sl->sp));
    memset(&sl->sm, 0, sizeof(sl->sm));
    for (size_t i = 0; i < b.st.size(); ++i) {
      sl->sp.st[i] = b.st[i];
      memcpy(sl->sm.m[2 * i], b.maps[i].m[0], 128);
      memcpy(sl->sm.m[2 * i + 1], b.maps[i].m[1], 128);
    }
    LaunchArgs& a = sl->a;
    memset(&a, 0, sizeof(a));
    a.nstages = (int)b.st.size();
    a.sync = sync;
    a.xstride = b.xstride();
    a.part_bytes = b.part_bytes();
    a.vec_bytes = b.vec_bytes();
    a.nslots = slots;
    a.slot_bytes = b.slot_bytes();
    a.grid = r.grid;
    a.smem = smem;
    delete g_cache[g_cache_next];
    g_cache[g_cache_next] = sl;
    g_cache_next = (g_cache_next + 1) % kLaunchCache;
  }
  LaunchArgs a = sl->a;
  a.small = &sl->sp;
  a.small_maps = &sl->sm;
  a.trace = r.set.trace_bytes >= (size_t)a.nstages * (size_t)a.grid * 128 ? r.set.trace : nullptr;
  a.wait_limit = r.set.wait_limit;
  a.stream = stream;
  cudaError_t e = sl->fn(a);
  if (e != cudaSuccess) return fail(FSVD_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  g_launches.fetch_add(1);
  return 0;
}

static void bump_generation() {   // call with g_set_mu held
  ++g_set.generation;
}

// y = (residual +) u(v(x)): the two stages of the low-rank projection, shared by the workspace
// and the built-in-scratch entry points (same K segments, same summation order).
static void build_lowrank(Builder& b, const void* x, const void* v, const void* u, const void* residual, void* y,
                          int d_in, int R, int d_out, void* partial) {
  {
    Stage& s = b.gemv(v, nullptr, R, d_in, d_in, true, 0, -1, true);
    b.vec(s, VL_SUM, x, d_in, 1, false);
    s.flags |= SF_IN_T;
    s.epi = EPI_PARTIAL;
    s.out = partial;
  }
  const int segs = b.st.back().segs;
  {
    Stage& s = b.gemv(u, nullptr, d_out, R, R, false);
    b.vec(s, VL_SUM, partial, R, segs, true);
    s.epi = residual ? EPI_RESID : EPI_STORE;
    s.resid = residual;
    s.flags |= SF_OUT_T | (residual ? SF_RESID_T : 0);
    s.out = y;
  }
}

// ------------------------------------------------------------------------------- C ABI
extern "C" {

int fsvd_version(void) { return 200; }
const char* fsvd_last_error_string(void) { return g_err; }
long long fsvd_launch_count(void) { return g_launches.load(); }

int fsvd_device_props(int* sm_count, int* smem_optin_bytes) {
  DevProps p;
  if (int e = get_props(p)) return e;
  if (sm_count) *sm_count = p.sms;
  if (smem_optin_bytes) *smem_optin_bytes = p.smem_optin;
  return 0;
}

int fsvd_set_trace_buffer(void* dev_ptr, size_t bytes) {
  current_settings();
  std::lock_guard<std::mutex> lock(g_set_mu);
  g_set.trace = reinterpret_cast<unsigned long long*>(dev_ptr);
  g_set.trace_bytes = dev_ptr ? bytes : 0;
  return 0;
}

int fsvd_set_launch_config(int warps, int depth, int grid) {
  current_settings();
  if (warps != 0 && warps != kConsumerWarps) return fail(FSVD_ERR_ARG, "warps must be 0 or %d", kConsumerWarps);
  if (depth < 0) return fail(FSVD_ERR_ARG, "depth (ring slots) must be >= 0");
  std::lock_guard<std::mutex> lock(g_set_mu);
  g_set.slots = depth;
  g_set.grid = grid < 0 ? 0 : grid;
  bump_generation();
  return 0;
}

int fsvd_set_wait_limit(long long sm_clocks) {
  current_settings();
  if (sm_clocks < 1000) return fail(FSVD_ERR_ARG, "the wait budget must be at least 1000 clocks");
  std::lock_guard<std::mutex> lock(g_set_mu);
  g_set.wait_limit = sm_clocks;
  return 0;
}

size_t fsvd_workspace_bytes(const fsvd_dims* dims) {
  if (!dims) return 0;
  if (use_tiles(*dims)) {   // tiled tensor-core path
    const size_t t = fsvd_tile_workspace_bytes(dims);
    // batches of 5..8: the per-op entry points use the single-launch kernel's layout on the same
    // workspace (both keep the status words first and their counters zero between launches)
    if (dims->B <= 8 && t) {
      const size_t s1 = ws_layout(*dims).total;
      return s1 > t ? s1 : t;
    }
    return t;
  }
  return ws_layout(*dims).total;
}

int fsvd_workspace_init(void* ws, size_t ws_bytes, void* stream) {
  if (!ws || ws_bytes < sizeof(SyncState)) return fail(FSVD_ERR_WORKSPACE, "workspace too small");
  CUDA_TRY(cudaMemsetAsync(ws, 0, ws_bytes, (cudaStream_t)stream));
  return 0;
}

int fsvd_workspace_status(void* ws, int* device_status) {
  if (!ws || !device_status) return fail(FSVD_ERR_ARG, "null argument");
  SyncState s;
  CUDA_TRY(cudaMemcpy(&s, ws, sizeof(s), cudaMemcpyDeviceToHost));
  *device_status = s.status;
  if (s.status == DS_CACHE_FULL)
    return fail(FSVD_ERR_CACHE_FULL, "a token arrived at a position beyond the cache (S_max): its key and value were not stored");
  if (s.status) return fail(FSVD_ERR_DEVICE_WAIT, "device wait ran out: code %d at stage %d", s.status, s.status_detail);
  return 0;
}

int fsvd_workspace_clear_status(void* ws, void* stream) {
  if (!ws) return fail(FSVD_ERR_ARG, "null argument");
  CUDA_TRY(cudaMemsetAsync(reinterpret_cast<char*>(ws) + offsetof(SyncState, status), 0, 2 * sizeof(int),
                           (cudaStream_t)stream));
  return 0;
}

static fsvd_dims op_dims(int dtype, int B) {
  fsvd_dims D;
  memset(&D, 0, sizeof(D));
  D.dtype = dtype;
  D.B = B;
  D.d = D.I = D.Rq = D.Rk = D.Rv = D.Ro = D.Rg = D.Ru = D.Rd = 8;
  D.H = D.Hk = 1;
  D.Dh = 64;
  D.S_max = 1;
  return D;
}

static int check_ws(const fsvd_dims& D, void* ws, size_t ws_bytes, WsLayout& L) {
  L = ws_layout(D);
  if (!ws) return fail(FSVD_ERR_WORKSPACE, "null workspace");
  if (!aligned16(ws)) return fail(FSVD_ERR_ALIGN, "workspace is not 16-byte aligned");
  if (ws_bytes < L.total) return fail(FSVD_ERR_WORKSPACE, "workspace of %zu bytes, %zu needed", ws_bytes, L.total);
  return 0;
}

int fsvd_lowrank_proj(const void* x, const void* v, const void* u, const void* residual, void* y,
                      int B, int d_in, int R, int d_out, int dtype, void* ws, size_t ws_bytes,
                      void* stream) {
  if (!x || !v || !u || !y) return fail(FSVD_ERR_ARG, "null argument");
  if (d_in <= 0 || R <= 0 || d_out <= 0 || d_in % 8 || R % 8)
    return fail(FSVD_ERR_ALIGN, "d_in=%d and R=%d must be positive multiples of 8", d_in, R);
  if (!aligned16(x) || !aligned16(v) || !aligned16(u) || !aligned16(y))
    return fail(FSVD_ERR_ALIGN, "pointers must be 16-byte aligned");
  if (dtype != FSVD_DTYPE_BF16 && dtype != FSVD_DTYPE_F32 && dtype != FSVD_DTYPE_BF16_Q4)
    return fail(FSVD_ERR_ARG, "bad dtype");
  fsvd_dims D = op_dims(dtype, B);
  D.Ro = R;
  WsLayout L;
  if (int e = check_ws(D, ws, ws_bytes, L)) return e;
  Resolved r;
  if (int e = resolve(dtype, B, r)) return e;
  Builder b(r, dtype, B);
  char* w = reinterpret_cast<char*>(ws);
  build_lowrank(b, x, v, u, residual, y, d_in, R, d_out, w + L.pb);
  return launch_small(r, b, reinterpret_cast<SyncState*>(w + L.sync), (cudaStream_t)stream);
}

int fsvd_lift(const void* p, const void* u, const void* residual, void* y, int B, int R, int d_out,
              int dtype, void* ws, size_t ws_bytes, void* stream) {
  if (!p || !u || !y) return fail(FSVD_ERR_ARG, "null argument");
  if (R <= 0 || d_out <= 0 || R % 8) return fail(FSVD_ERR_ALIGN, "R=%d must be a positive multiple of 8", R);
  if (!aligned16(p) || !aligned16(u) || !aligned16(y)) return fail(FSVD_ERR_ALIGN, "pointers must be 16-byte aligned");
  if (dtype != FSVD_DTYPE_BF16 && dtype != FSVD_DTYPE_F32 && dtype != FSVD_DTYPE_BF16_Q4)
    return fail(FSVD_ERR_ARG, "bad dtype");
  fsvd_dims D = op_dims(dtype, B);
  WsLayout L;
  if (int e = check_ws(D, ws, ws_bytes, L)) return e;
  Resolved r;
  if (int e = resolve(dtype, B, r)) return e;
  Builder b(r, dtype, B);
  char* w = reinterpret_cast<char*>(ws);
  Stage& s = b.gemv(u, nullptr, d_out, R, R, false);
  b.vec(s, VL_SUM, p, R, 1, false);
  s.flags |= SF_IN_T | SF_OUT_T | (residual ? SF_RESID_T : 0);
  s.epi = residual ? EPI_RESID : EPI_STORE;
  s.resid = residual;
  s.out = y;
  return launch_small(r, b, reinterpret_cast<SyncState*>(w + L.sync), (cudaStream_t)stream);
}

int fsvd_mlp_swiglu_decode(const void* x, const void* norm_w, float eps, const void* upgate_v,
                           const void* gate_u, const void* up_u, const void* down_v,
                           const void* down_u, const void* residual, void* y, int B, int d, int I,
                           int Ru, int Rg, int Rd, int dtype, void* ws, size_t ws_bytes,
                           void* stream) {
  if (!x || !gate_u || !up_u || !down_v || !down_u || !y) return fail(FSVD_ERR_ARG, "null argument");
  if (dtype != FSVD_DTYPE_BF16 && dtype != FSVD_DTYPE_F32 && dtype != FSVD_DTYPE_BF16_Q4)
    return fail(FSVD_ERR_ARG, "bad dtype");
  if (d <= 0 || I <= 0 || Ru <= 0 || Rg <= 0 || Rd <= 0 || d % 8 || I % 8 || Ru % 8 || Rg % 8 || Rd % 8)
    return fail(FSVD_ERR_ALIGN, "d, I and the ranks must be positive multiples of 8");
  if (Ru != Rg) return fail(FSVD_ERR_UNSUPPORTED, "gate and up ranks must match (Rg=%d, Ru=%d)", Rg, Ru);
  const void* ps[] = {x, gate_u, up_u, down_v, down_u, y};
  for (const void* p : ps)
    if (!aligned16(p)) return fail(FSVD_ERR_ALIGN, "pointers must be 16-byte aligned");
  fsvd_dims D = op_dims(dtype, B);
  D.d = d; D.I = I; D.Ru = Ru; D.Rg = Rg; D.Rd = Rd;
  WsLayout L;
  if (int e = check_ws(D, ws, ws_bytes, L)) return e;
  Resolved r;
  if (int e = resolve(dtype, B, r)) return e;
  Builder b(r, dtype, B);
  char* w = reinterpret_cast<char*>(ws);
  int segs_rank = 1;
  const void* pcat = x;
  bool pcat_T = true;
  if (upgate_v) {
    Stage& s = b.gemv(upgate_v, nullptr, Ru + Rg, d, d, true);
    b.vec(s, norm_w ? VL_RMSNORM : VL_SUM, x, d, 1, false);
    s.flags |= SF_IN_T;
    s.vl_w = norm_w;
    s.eps = eps;
    s.epi = EPI_PARTIAL;
    s.out = w + L.pa;
    segs_rank = s.segs;
    pcat = w + L.pa;
    pcat_T = false;
  }
  {
    Stage& s = b.gemv(gate_u, up_u, I, Rg, Rg, false);
    if (pcat_T) {
      b.vec(s, VL_SUM, pcat, Ru + Rg, 1, false);
      s.flags |= SF_IN_T;
    } else {
      b.vec(s, VL_SUM, pcat, Ru + Rg, segs_rank, true);
    }
    s.xA_off = Ru;
    s.xB_off = 0;
    s.epi = EPI_SWIGLU;
    s.flags |= SF_OUT_T;
    s.out = w + L.hact;
  }
  {
    Stage& s = b.gemv(down_v, nullptr, Rd, I, I, true, 0, -1, true);
    b.vec(s, VL_SUM, w + L.hact, I, 1, true);
    s.flags |= SF_IN_T;
    s.epi = EPI_PARTIAL;
    s.out = w + L.pb;
  }
  const int segs = b.st.back().segs;
  {
    Stage& s = b.gemv(down_u, nullptr, d, Rd, Rd, false);
    b.vec(s, VL_SUM, w + L.pb, Rd, segs, true);
    s.epi = residual ? EPI_RESID : EPI_STORE;
    s.resid = residual;
    s.flags |= SF_OUT_T | (residual ? SF_RESID_T : 0);
    s.out = y;
  }
  return launch_small(r, b, reinterpret_cast<SyncState*>(w + L.sync), (cudaStream_t)stream);
}

int fsvd_qkv_rope_append(const void* x, const void* norm_w, float eps, const void* qkv_v,
                         const void* q_u, const void* k_u, const void* v_u, const void* cos_tab,
                         const void* sin_tab, void* k_cache, void* v_cache,
                         const int* cache_seqlens, void* q_out, int B, int d, int H, int Hk, int Dh,
                         int Rq, int Rk, int Rv, int S_max, int dtype, void* ws, size_t ws_bytes,
                         void* stream) {
  if (!x || !qkv_v || !q_u || !k_u || !v_u || !cos_tab || !sin_tab || !k_cache || !v_cache ||
      !cache_seqlens || !q_out)
    return fail(FSVD_ERR_ARG, "null argument");
  fsvd_dims D = op_dims(dtype, B);
  D.d = d; D.H = H; D.Hk = Hk; D.Dh = Dh; D.Rq = Rq; D.Rk = Rk; D.Rv = Rv; D.S_max = S_max;
  if (int e = check_dims(D)) return e;
  const void* ps[] = {x, qkv_v, q_u, k_u, v_u, k_cache, v_cache, q_out};
  for (const void* p : ps)
    if (!aligned16(p)) return fail(FSVD_ERR_ALIGN, "pointers must be 16-byte aligned");
  WsLayout L;
  if (int e = check_ws(D, ws, ws_bytes, L)) return e;
  Resolved r;
  if (int e = resolve(dtype, B, r)) return e;
  Builder b(r, dtype, B);
  char* w = reinterpret_cast<char*>(ws);
  const int half = Dh / 2, Rqkv = Rq + Rk + Rv;
  {
    Stage& s = b.gemv(qkv_v, nullptr, Rqkv, d, d, true);
    b.vec(s, norm_w ? VL_RMSNORM : VL_SUM, x, d, 1, false);
    s.flags |= SF_IN_T;
    s.vl_w = norm_w;
    s.eps = eps;
    s.epi = EPI_PARTIAL;
    s.out = w + L.pa;
  }
  const int segs = b.st.back().segs;
  {
    Stage& s = b.gemv(q_u, b.row_ptr(q_u, half, Rq), H * half, Rq, Rq, false, half);
    b.vec(s, VL_SUM, w + L.pa, Rqkv, segs, true);
    s.rope_half = half;
    s.epi = EPI_ROPE_Q;
    s.flags |= SF_OUT_T;
    s.out = q_out;
    s.cos_tab = cos_tab; s.sin_tab = sin_tab; s.seqlens = cache_seqlens;
    s.H = H; s.Hk = Hk; s.Dh = Dh; s.S_max = S_max;
  }
  {
    Stage& s = b.gemv(k_u, b.row_ptr(k_u, half, Rk), Hk * half, Rk, Rk, false, half);
    s.rope_half = half;
    s.xA_off = s.xB_off = Rq;
    s.epi = EPI_ROPE_K;
    s.cache = k_cache;
    s.cos_tab = cos_tab; s.sin_tab = sin_tab; s.seqlens = cache_seqlens;
    s.H = H; s.Hk = Hk; s.Dh = Dh; s.S_max = S_max;
  }
  {
    Stage& s = b.gemv(v_u, nullptr, Hk * Dh, Rv, Rv, false);
    s.xA_off = Rq + Rk;
    s.epi = EPI_V;
    s.cache = v_cache;
    s.seqlens = cache_seqlens;
    s.H = H; s.Hk = Hk; s.Dh = Dh; s.S_max = S_max;
  }
  return launch_small(r, b, reinterpret_cast<SyncState*>(w + L.sync), (cudaStream_t)stream);
}

int fsvd_flash_decode(const void* q, const void* k_cache, const void* v_cache,
                      const int* cache_seqlens, int seqlen_add, void* out, int B, int H, int Hk,
                      int Dh, int S_max, float scale, int dtype, void* ws, size_t ws_bytes,
                      void* stream) {
  if (!q || !k_cache || !v_cache || !cache_seqlens || !out) return fail(FSVD_ERR_ARG, "null argument");
  fsvd_dims D = op_dims(dtype, B);
  D.H = H; D.Hk = Hk; D.Dh = Dh; D.S_max = S_max;
  if (int e = check_dims(D)) return e;
  WsLayout L;
  if (int e = check_ws(D, ws, ws_bytes, L)) return e;
  Resolved r;
  if (int e = resolve(dtype, B, r)) return e;
  Builder b(r, dtype, B);
  char* w = reinterpret_cast<char*>(ws);
  Stage s = b.blank();
  s.type = ST_ATTN;
  s.flags = SF_IN_T | SF_OUT_T;
  s.q = q;
  s.kcache = k_cache;
  s.vcache = v_cache;
  s.seqlens = cache_seqlens;
  s.seqlen_add = seqlen_add;
  s.out = out;
  s.part_acc = reinterpret_cast<float*>(w + L.part_acc);
  s.part_ml = reinterpret_cast<float*>(w + L.part_ml);
  s.counters = reinterpret_cast<int*>(w + L.counters);
  s.H = H; s.Hk = Hk; s.Dh = Dh; s.S_max = S_max;
  s.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)Dh);
  b.attn_geometry(s);
  b.push(s);
  return launch_small(r, b, reinterpret_cast<SyncState*>(w + L.sync), (cudaStream_t)stream);
}

int fsvd_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab,
                      const void* sin_tab, const int* cache_seqlens, const void* x_in, void* x_out,
                      void* ws, size_t ws_bytes, void* stream) {
  if (!dims || !layer || !cos_tab || !sin_tab || !cache_seqlens || !x_in || !x_out)
    return fail(FSVD_ERR_ARG, "null argument");
  const fsvd_dims& D = *dims;
  if (use_tiles(D)) {
    // batches of 9..128 sequences: tiled GEMMs on tcgen05 (fsvd_tile.cu), several launches
    if (int e = check_layer_ptrs(*layer)) return e;
    if (!aligned16(ws)) return fail(FSVD_ERR_ALIGN, "workspace is not 16-byte aligned");
    return fsvd_tile_decode_layer(dims, layer, cos_tab, sin_tab, cache_seqlens, x_in, x_out, ws, ws_bytes,
                                  current_settings().wait_limit, stream);
  }
  if (int e = check_dims(D)) return e;
  if (int e = check_layer_ptrs(*layer)) return e;
  WsLayout L;
  if (int e = check_ws(D, ws, ws_bytes, L)) return e;
  Resolved r;
  if (int e = resolve(D.dtype, D.B, r)) return e;
  Builder b(r, D.dtype, D.B);
  LayerIO io = {x_in, false, x_out, cache_seqlens, cos_tab, sin_tab};
  build_layer(b, D, *layer, io, reinterpret_cast<char*>(ws), L);
  return launch_small(r, b, reinterpret_cast<SyncState*>(reinterpret_cast<char*>(ws) + L.sync),
                      (cudaStream_t)stream);
}

// Tensor-parallel layer on the rank's shards (fsvd_tile.cu; exchange protocol in fsvd_exchange.h).
size_t fsvd_tp_workspace_bytes(const fsvd_dims* dims) { return fsvd_tile_workspace_bytes(dims); }

int fsvd_tp_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab, const void* sin_tab,
                         const int* cache_seqlens, const void* x_in, const void* x_norm_in, void* x_out,
                         const void* next_norm_w, void* x_norm_out, fsvd_exchange* ex, void* ws, size_t ws_bytes,
                         void* stream) {
  if (!dims || !layer || !cos_tab || !sin_tab || !cache_seqlens || !x_in || !x_out || !ex)
    return fail(FSVD_ERR_ARG, "null argument");
  if (int e = check_layer_ptrs(*layer)) return e;
  if (!aligned16(ws)) return fail(FSVD_ERR_ALIGN, "workspace is not 16-byte aligned");
  return fsvd_tile_tp_decode_layer(dims, layer, cos_tab, sin_tab, cache_seqlens, x_in, x_norm_in, x_out, next_norm_w,
                                   x_norm_out, ex, ws, ws_bytes, current_settings().wait_limit, stream);
}

// ------------------------------------------------------------------------------- model
struct fsvd_model {
  fsvd_dims D;
  Resolved r;
  WsLayout L;
  char* ws = nullptr;
  Stage* prog = nullptr;
  unsigned char* maps = nullptr;   // TMA descriptors, 2 x 128 bytes per stage
  int nstages = 0, nbarriers = 0, xstride = 0, max_steps = 0, part_bytes = 0, vec_bytes = 0, nslots = 0, slot_bytes = 0;
  size_t smem = 0;
  int* tokens = nullptr;
  int* seqlens = nullptr;
  int* token_log = nullptr;
  int* step_counter = nullptr;
  float* logits = nullptr;
  float* xbuf = nullptr;  // hidden state between layers, [B, d] of type T
  char* extra = nullptr;
  fsvd_tile_model* tile = nullptr;   // batches above 8: the tiled path owns everything
};

int fsvd_model_destroy(fsvd_model* m);

int fsvd_model_create(const fsvd_dims* dims, const fsvd_layer* layers, const void* embed,
                      const void* final_norm_w, const void* lm_head, const void* cos_tab,
                      const void* sin_tab, int max_steps, fsvd_model** out) {
  if (!dims || !layers || !embed || !final_norm_w || !lm_head || !cos_tab || !sin_tab || !out)
    return fail(FSVD_ERR_ARG, "null argument");
  const fsvd_dims& D = *dims;
  if (use_tiles(D)) {
    for (int l = 0; l < D.n_layers; ++l)
      if (int e = check_layer_ptrs(layers[l])) return e;
    if (!aligned16(embed) || !aligned16(lm_head) || !aligned16(final_norm_w))
      return fail(FSVD_ERR_ALIGN, "embed / lm_head / norm pointers must be 16-byte aligned");
    fsvd_tile_model* t = nullptr;
    if (int e = fsvd_tile_model_create(dims, layers, embed, final_norm_w, lm_head, cos_tab, sin_tab, max_steps,
                                       current_settings().wait_limit, &t))
      return e;
    fsvd_model* m = new fsvd_model();
    m->D = D;
    m->tile = t;
    m->max_steps = max_steps;
    *out = m;
    return 0;
  }
  if (int e = check_dims(D)) return e;
  if (D.n_layers < 1 || D.vocab < 1) return fail(FSVD_ERR_ARG, "n_layers=%d vocab=%d", D.n_layers, D.vocab);
  for (int l = 0; l < D.n_layers; ++l)
    if (int e = check_layer_ptrs(layers[l])) return e;
  if (!aligned16(embed) || !aligned16(lm_head) || !aligned16(final_norm_w))
    return fail(FSVD_ERR_ALIGN, "embed / lm_head / norm pointers must be 16-byte aligned");
  if (max_steps < 1) max_steps = 1;

  fsvd_model* m = new fsvd_model();
  m->D = D;
  m->max_steps = max_steps;
  m->L = ws_layout(D);
  if (int e = resolve(D.dtype, D.B, m->r)) { delete m; return e; }

  const size_t extra_bytes = al256((size_t)D.B * 4) * 2 + al256(4) + al256((size_t)max_steps * D.B * 4) +
                             al256((size_t)D.B * D.vocab * 4);
  cudaError_t ce = cudaMalloc(&m->ws, m->L.total);
  if (ce == cudaSuccess) ce = cudaMalloc(&m->extra, extra_bytes);
  if (ce == cudaSuccess) ce = cudaMemset(m->ws, 0, m->L.total);
  if (ce == cudaSuccess) ce = cudaMemset(m->extra, 0, extra_bytes);
  if (ce != cudaSuccess) {
    cudaFree(m->ws); cudaFree(m->extra); delete m;
    return fail(FSVD_ERR_CUDA, "allocating model scratch failed: %s", cudaGetErrorString(ce));
  }
  size_t o = 0;
  m->tokens = reinterpret_cast<int*>(m->extra + o);        o += al256((size_t)D.B * 4);
  m->seqlens = reinterpret_cast<int*>(m->extra + o);       o += al256((size_t)D.B * 4);
  m->step_counter = reinterpret_cast<int*>(m->extra + o);  o += al256(4);
  m->token_log = reinterpret_cast<int*>(m->extra + o);     o += al256((size_t)max_steps * D.B * 4);
  m->logits = reinterpret_cast<float*>(m->extra + o);

  Builder b(m->r, D.dtype, D.B);
  // The hidden state ping-pongs between two fp32 buffers: `hidden` (between the halves of a
  // layer) and `xbuf` (between layers), so a residual never reads what its stage overwrites.
  float* xbuf = nullptr;
  ce = cudaMalloc(&xbuf, al256((size_t)D.B * D.d * 8));
  if (ce == cudaSuccess) ce = cudaMemset(xbuf, 0, al256((size_t)D.B * D.d * 8));
  if (ce != cudaSuccess) {
    cudaFree(m->ws); cudaFree(m->extra); delete m;
    return fail(FSVD_ERR_CUDA, "allocating model scratch failed: %s", cudaGetErrorString(ce));
  }
  {
    Stage s = b.blank();
    s.type = ST_EMBED;
    s.WA = embed;
    s.P = D.d;
    s.out = xbuf;
    s.flags = SF_OUT_T;
    s.tokens = m->tokens;
    s.vocab = D.vocab;
    b.push(s);
  }
  for (int l = 0; l < D.n_layers; ++l) {
    LayerIO io = {xbuf, true, xbuf, m->seqlens, cos_tab, sin_tab};
    build_layer(b, D, layers[l], io, m->ws, m->L);
  }
  {
    Stage& s = b.gemv(lm_head, nullptr, D.vocab, D.d, D.d, false, 0, 0);   // lm_head stays dense
    b.vec(s, VL_RMSNORM, xbuf, D.d, 1, true);
    s.flags |= SF_IN_T;
    s.vl_w = final_norm_w;
    s.eps = D.eps;
    s.epi = EPI_STORE;
    s.out = m->logits;
  }
  {
    Stage s = b.blank();
    s.type = ST_ARGMAX;
    s.flags = 0;
    s.vl_src = m->logits;
    s.vocab = D.vocab;
    s.tokens = m->tokens;
    s.token_log = m->token_log;
    s.step_counter = m->step_counter;
    s.seqlens_rw = m->seqlens;
    s.max_steps = max_steps;
    b.push(s);
    b.need_barrier(b.st.back());
  }
  int pe = plan_smem(m->r, b, m->nslots, m->smem);
  if (!pe) pe = encode_all(b);
  if (pe) {
    cudaFree(m->ws); cudaFree(m->extra); cudaFree(xbuf); delete m;
    return pe;
  }
  m->nstages = (int)b.st.size();
  for (const Stage& s : b.st) m->nbarriers += (s.flags & SF_BARRIER) ? 1 : 0;
  m->xstride = b.xstride();
  m->part_bytes = b.part_bytes();
  m->vec_bytes = b.vec_bytes();
  m->slot_bytes = b.slot_bytes();
  static_assert(sizeof(MapPair) == 256, "two descriptors per stage");
  ce = cudaMalloc(&m->prog, sizeof(Stage) * b.st.size());
  if (ce == cudaSuccess) ce = cudaMalloc(&m->maps, sizeof(MapPair) * b.maps.size());
  if (ce == cudaSuccess)
    ce = cudaMemcpy(m->prog, b.st.data(), sizeof(Stage) * b.st.size(), cudaMemcpyHostToDevice);
  if (ce == cudaSuccess)
    ce = cudaMemcpy(m->maps, b.maps.data(), sizeof(MapPair) * b.maps.size(), cudaMemcpyHostToDevice);
  if (ce != cudaSuccess) {
    cudaFree(m->ws); cudaFree(m->extra); cudaFree(xbuf); cudaFree(m->prog); cudaFree(m->maps); delete m;
    return fail(FSVD_ERR_CUDA, "uploading the stage program failed: %s", cudaGetErrorString(ce));
  }
  m->xbuf = xbuf;
  *out = m;
  return 0;
}

int fsvd_model_destroy(fsvd_model* m) {
  if (!m) return 0;
  if (m->tile) fsvd_tile_model_destroy(m->tile);
  cudaFree(m->ws);
  cudaFree(m->extra);
  cudaFree(m->prog);
  cudaFree(m->maps);
  cudaFree(m->xbuf);
  delete m;
  return 0;
}

int fsvd_model_step(fsvd_model* m, int n_steps, void* stream) {
  if (!m) return fail(FSVD_ERR_ARG, "null model");
  if (m->tile) return fsvd_tile_model_step(m->tile, n_steps, stream);
  SyncState* sync = reinterpret_cast<SyncState*>(m->ws + m->L.sync);
  const Settings set = current_settings();   // the geometry is the one of fsvd_model_create
  for (int i = 0; i < n_steps; ++i) {
    LaunchArgs a;
    memset(&a, 0, sizeof(a));
    a.prog = m->prog;
    a.maps = m->maps;
    a.nstages = m->nstages;
    a.sync = sync;
    a.xstride = m->xstride;
    a.part_bytes = m->part_bytes;
    a.vec_bytes = m->vec_bytes;
    a.nslots = m->nslots;
    a.slot_bytes = m->slot_bytes;
    a.trace = set.trace_bytes >= (size_t)m->nstages * m->r.grid * 128 ? set.trace : nullptr;
    a.wait_limit = set.wait_limit;
    a.grid = m->r.grid;
    a.smem = m->smem;
    a.stream = (cudaStream_t)stream;
    cudaError_t e = m->r.fn(a);
    if (e != cudaSuccess) return fail(FSVD_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    g_launches.fetch_add(1);
  }
  return 0;
}

int fsvd_model_buffers(fsvd_model* m, int** tokens, int** seqlens, int** token_log,
                       int** step_counter, float** logits, float** hidden) {
  if (!m) return fail(FSVD_ERR_ARG, "null model");
  if (m->tile) {
    fsvd_tile_model_buffers(m->tile, tokens, seqlens, token_log, step_counter, logits, hidden);
    return 0;
  }
  if (tokens) *tokens = m->tokens;
  if (seqlens) *seqlens = m->seqlens;
  if (token_log) *token_log = m->token_log;
  if (step_counter) *step_counter = m->step_counter;
  if (logits) *logits = m->logits;
  if (hidden) *hidden = m->xbuf;
  return 0;
}

int fsvd_model_num_stages(fsvd_model* m) { return !m ? 0 : m->tile ? fsvd_tile_model_launches_per_step(m->tile) : m->nstages; }
int fsvd_model_num_barriers(fsvd_model* m) { return (m && !m->tile) ? m->nbarriers : 0; }

int fsvd_model_status(fsvd_model* m, int* device_status) {
  if (!m) return fail(FSVD_ERR_ARG, "null model");
  return fsvd_workspace_status(m->tile ? fsvd_tile_model_ws(m->tile) : m->ws, device_status);
}

int fsvd_model_reset_sync(fsvd_model* m, void* stream) {
  if (!m) return fail(FSVD_ERR_ARG, "null model");
  if (m->tile) return fsvd_tile_model_reset(m->tile, stream);
  CUDA_TRY(cudaMemsetAsync(m->ws + m->L.sync, 0, sizeof(SyncState), (cudaStream_t)stream));
  CUDA_TRY(cudaMemsetAsync(m->ws + m->L.counters, 0, kCounterBytes, (cudaStream_t)stream));
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------- built-in scratch
// fsvd_lowrank_proj_static: the low-rank projection on scratch that is part of the library
// image instead of a caller-provided workspace.  The scratch holds the grid-barrier words and the
// rank-space partial sums [segments][B][R] in fp32; one array per device, shared by every call.
constexpr int kStaticMaxBR = 8192;  // limit on B * R
constexpr size_t kStaticSyncBytes = 256;
constexpr size_t kStaticScratchBytes = kStaticSyncBytes + (size_t)kMaxSegs * kStaticMaxBR * sizeof(float);
static_assert(sizeof(SyncState) <= kStaticSyncBytes, "barrier words must fit the scratch header");
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static void* g_static_ptr[16] = {nullptr};
static std::mutex g_static_mu;

// Device address of the scratch on the current device.  The first call on a device looks the
// address up and clears the barrier words (the only part that has to start at zero: the partial
// sums are fully rewritten by every call, the barrier counters only ever grow).
static int static_scratch(char** out, cudaStream_t stream) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 16) return fail(FSVD_ERR_UNSUPPORTED, "device ordinal %d unsupported (0..15)", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    if (!p) return fail(FSVD_ERR_CUDA, "built-in scratch has no device address");
    CUDA_TRY(cudaMemsetAsync(p, 0, kStaticSyncBytes, stream));
    g_static_ptr[dev] = p;
  }
  *out = reinterpret_cast<char*>(g_static_ptr[dev]);
  return 0;
}

extern "C" int fsvd_lowrank_proj_static(const void* x, const void* v, const void* u,
                                        const void* residual, void* y, int B, int d_in, int R,
                                        int d_out, int dtype, void* stream) {
  if (!x || !v || !u || !y) return fail(FSVD_ERR_ARG, "null argument");
  if (d_in <= 0 || R <= 0 || d_out <= 0 || d_in % 8 || R % 8)
    return fail(FSVD_ERR_ALIGN, "d_in=%d and R=%d must be positive multiples of 8", d_in, R);
  if (!aligned16(x) || !aligned16(v) || !aligned16(u) || !aligned16(y))
    return fail(FSVD_ERR_ALIGN, "pointers must be 16-byte aligned");
  if (dtype != FSVD_DTYPE_BF16 && dtype != FSVD_DTYPE_F32) return fail(FSVD_ERR_ARG, "bad dtype");
  Resolved r;
  if (int e = resolve(dtype, B, r)) return e;
  if ((long long)B * R > kStaticMaxBR)
    return fail(FSVD_ERR_WORKSPACE,
                "B*R = %lld exceeds the built-in scratch (B*R <= %d); use fsvd_lowrank_proj with a workspace",
                (long long)B * R, kStaticMaxBR);
  char* w = nullptr;
  if (int e = static_scratch(&w, (cudaStream_t)stream)) return e;
  float* partial = reinterpret_cast<float*>(w + kStaticSyncBytes);
  Builder b(r, dtype, B);
  build_lowrank(b, x, v, u, residual, y, d_in, R, d_out, partial);
  if (b.st[0].segs > kMaxSegs) return fail(FSVD_ERR_UNSUPPORTED, "%d K segments exceed the built-in scratch", b.st[0].segs);
  return launch_small(r, b, reinterpret_cast<SyncState*>(w), (cudaStream_t)stream);
}

// Waits for the stream's work on the built-in scratch, then reads its device status the way
// fsvd_workspace_status does; `reset` != 0 also zeroes the barrier words and the status (after a
// wait that ran out the arrival count of the abandoned launch is left behind).
extern "C" int fsvd_static_status(int* device_status, int reset) {
  if (!device_status) return fail(FSVD_ERR_ARG, "null argument");
  char* w = nullptr;
  if (int e = static_scratch(&w, nullptr)) return e;
  CUDA_TRY(cudaDeviceSynchronize());
  const int rc = fsvd_workspace_status(w, device_status);
  if (reset) {
    CUDA_TRY(cudaMemset(w, 0, kStaticSyncBytes));
  }
  return rc;
}

// Launches a one-stage program whose stage stands behind a grid barrier that no stage arrives at:
// every CTA waits, gives up after the wait budget (fsvd_set_wait_limit) and returns; the stage itself copies nothing.  The
// launch returns 0; the status words then hold DS_BARRIER_TIMEOUT with stage index 0.  Used by the
// tests to see a wait run out within its budget without anything hanging.
extern "C" int fsvd_selftest_wait_timeout(void* ws, size_t ws_bytes, void* stream) {
  if (!ws || ws_bytes < sizeof(SyncState)) return fail(FSVD_ERR_WORKSPACE, "workspace too small");
  Resolved r;
  if (int e = resolve(FSVD_DTYPE_BF16, 1, r)) return e;
  r.set.trace = nullptr;
  r.set.trace_bytes = 0;
  Builder b(r, FSVD_DTYPE_BF16, 1);
  char* w = reinterpret_cast<char*>(ws);
  Stage s = b.blank();
  s.type = ST_EMBED;
  s.P = 0;   // zero elements to copy
  s.vocab = 1;
  s.flags = SF_OUT_T | SF_BARRIER;
  b.push(s);
  return launch_small(r, b, reinterpret_cast<SyncState*>(w), (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------- int4 tile streams
// Repacks one PackedQuantLinear (qweight uint8 [rows, K/2], low nibble = even input; scales fp16
// [rows, ceil(K/128)]; zeros int16, all 8 for the symmetric format) into the tile stream the
// kernel reads (fsvd_stage.h).  One thread writes one 16-byte word of the stream.
__device__ int g_q4_bad_zero;

__global__ void q4_pack_kernel(const unsigned char* __restrict__ qweight, const unsigned short* __restrict__ scales,
                               const short* __restrict__ zeros, int rows, int K, int nct, long long nwords,
                               uint4* __restrict__ out) {
  const long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= nwords) return;
  const int w16 = (int)(w % 32);
  const long long trow = w / 32;
  const int r17 = (int)(trow % kQ4TileRows);
  const long long tile = trow / kQ4TileRows;
  const int ct = (int)(tile % nct);
  const long long rt = tile / nct;
  const int G = (K + kQ4Group - 1) / kQ4Group, rowbytes = K / 2;
  union {
    uint4 v;
    unsigned char b[16];
    unsigned short h[8];
    unsigned int u[4];
  } o;
  if (r17 < kUnitRows) {
    const long long row = rt * kUnitRows + r17;
    for (int i = 0; i < 16; ++i) {
      const int bcol = ct * kQ4RowBytes + w16 * 16 + i;
      o.b[i] = (row < rows && bcol < rowbytes) ? qweight[row * rowbytes + bcol] : (unsigned char)0x88;
    }
    // inside every 32-bit word (inputs 8 i .. 8 i + 7): even inputs to the low half, odd inputs to
    // the high half, so that (w >> 4 n) & 0x000f000f is the pair of inputs (2 n, 2 n + 1)
    for (int i = 0; i < 4; ++i) {
      const unsigned int w = o.u[i];
      unsigned int r = 0;
      for (int n = 0; n < 4; ++n) {
        r |= ((w >> (8 * n)) & 0xfu) << (4 * n);             // input 2 n
        r |= ((w >> (8 * n + 4)) & 0xfu) << (16 + 4 * n);    // input 2 n + 1
      }
      o.u[i] = r;
    }
  } else {
    const long long row = rt * kUnitRows + w16;
    for (int j = 0; j < 8; ++j) {
      const int gi = ct * 8 + j;
      const bool in = w16 < kUnitRows && row < rows && gi < G;
      o.h[j] = in ? scales[row * G + gi] : (unsigned short)0;
      if (in && zeros && zeros[row * G + gi] != 8) atomicOr(&g_q4_bad_zero, 1);
    }
  }
  out[w] = o.v;
}

extern "C" size_t fsvd_q4_packed_bytes(int rows, int K) {
  if (rows < 1 || K < 1) return 0;
  return q4_bytes(rows, K);
}

extern "C" int fsvd_q4_pack(const void* qweight, const void* scales, const void* zeros, int rows, int K,
                            void* out, void* stream) {
  if (!qweight || !scales || !out) return fail(FSVD_ERR_ARG, "null argument");
  if (rows < 1 || K < 8 || K % 8) return fail(FSVD_ERR_ALIGN, "K=%d must be a positive multiple of 8", K);
  if (!aligned16(out)) return fail(FSVD_ERR_ALIGN, "the tile stream must start on a 16-byte boundary");
  const int nct = (K + kQ4BoxCols - 1) / kQ4BoxCols;
  const long long nwords = (long long)(q4_bytes(rows, K) / 16);
  cudaStream_t st = (cudaStream_t)stream;
  const int zero = 0;
  if (zeros) CUDA_TRY(cudaMemcpyToSymbolAsync(g_q4_bad_zero, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st));
  q4_pack_kernel<<<(unsigned)((nwords + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const unsigned char*>(qweight), reinterpret_cast<const unsigned short*>(scales),
      reinterpret_cast<const short*>(zeros), rows, K, nct, nwords, reinterpret_cast<uint4*>(out));
  CUDA_TRY(cudaGetLastError());
  if (zeros) {
    int bad = 0;
    CUDA_TRY(cudaMemcpyFromSymbolAsync(&bad, g_q4_bad_zero, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    if (bad) return fail(FSVD_ERR_UNSUPPORTED, "only the symmetric int4 format (every zero point = 8) is supported");
  }
  return 0;
}
