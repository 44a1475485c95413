// Stage program shared by the host-side program builder and the device interpreter.
//
// One decode step is a short program of dependent stages (rank projection, lift with a
// fused epilogue, split-KV attention, ...).  A single persistent kernel, one CTA per SM,
// walks the program.  The factor matrices of all GEMV stages form one long stream of 7 KB
// boxes (16 rows x 448 bytes) per CTA; producer warps copy the boxes with TMA into a
// shared-memory ring, in program order and as far ahead as the ring allows.  The addresses of
// the factors do not depend on the activations, so the stream keeps running while the consumer
// warps wait at the grid barrier between two stages.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define FSVD_HD __host__ __device__
#else
#define FSVD_HD
#endif

namespace fsvd {

enum StageType : int {
  ST_END = 0,
  ST_GEMV = 1,    // y = W x, rows split over warps, optional K split into partial sums
  ST_ATTN = 2,    // split-KV single-query attention over the dense cache + ordered combine
  ST_EMBED = 3,   // hidden[b,:] = embed[token[b],:]
  ST_ARGMAX = 4,  // token[b] = argmax_v logits[b,v]; advances seqlens / step counter
};

enum Epilogue : int {
  EPI_PARTIAL = 0,  // out[(seg*B+b)*P + p] = acc            (fp32, summed by the consumer)
  EPI_STORE = 1,    // out[b*P + p] = rnd(acc)               (fp32 container or T, see OUT_T)
  EPI_RESID = 2,    // out[b*P + p] = rnd(resid[b*P+p] + rnd(acc))
  EPI_SWIGLU = 3,   // out[b*P + p] = rnd(rnd(silu(rnd(accA))) * rnd(accB))   A=gate, B=up
  EPI_ROPE_Q = 4,   // rotate (accA, accB) = dims (j, j+half) of a head, store to q buffer
  EPI_ROPE_K = 5,   // same rotation, store into the key cache at position seqlens[b]
  EPI_V = 6,        // store rnd(acc) into the value cache at position seqlens[b]
  EPI_QKV = 7,      // q, k and v lifts in one stage over the packed [q_u; k_u; v_u] matrix: logical rows
                    // [0, H*half) are ROPE_Q, the next Hk*half ROPE_K (cache), the last Hk*half the
                    // value row halves (vcache); the input of part i starts at element i * K
};

enum VecLoad : int {
  VL_NONE = 0,     // keep the vector already staged in shared memory
  VL_SUM = 1,      // x[b,k] = rnd(sum_s src[(s*B+b)*len + k])
  VL_RMSNORM = 2,  // x[b,:] = rnd(w * rnd(src[b,:] * rsqrt(mean(src[b,:]^2) + eps)))
};

enum StageFlags : int {
  SF_BARRIER = 1,    // grid-wide barrier before this stage: waits for every warp's SF_ARRIVE
  SF_IN_T = 2,       // vl_src (or q for ST_ATTN) holds T instead of fp32
  SF_OUT_T = 4,      // out holds T instead of fp32
  SF_RESID_T = 8,    // resid holds T instead of fp32
  SF_ARRIVE = 16,    // arrive at the grid barrier after this stage (the next one has SF_BARRIER)
  SF_Q4 = 32,        // WA / WB are int4 tile streams (see kQ4*), activations stay T = bf16
  SF_SHARED_CACHE = 128,  // the B rows are consecutive positions of one sequence: all use cache row 0
  SF_SEG_X = 64,     // segs divides the grid, so a CTA's units all lie in K segment (first unit % segs):
                     // only that segment of the input (a T vector) is staged, at offset 0
};

// `rnd` above rounds to the storage type T (bf16) and is the identity when T is fp32: these
// are the points at which the PyTorch low-rank path materialises a tensor in the model dtype.
struct alignas(16) Stage {
  int type, flags, epi, vl_mode;
  const void* WA;        // [rows, ldw] row-major factor (nn.Linear weight layout), type T
  const void* WB;        // second operand group (up factor / second rotary half) or null
  int P;                 // logical rows (a logical row owns one A row and, if WB, one B row)
  int K;                 // reduction length
  int ldw;               // row stride of WA/WB in elements
  int segs;              // number of K segments (partial sums) per row group
  int kseg;              // elements per K segment (cps boxes)
  int xA_off, xB_off;    // offset of the operand-group input inside the staged vector
  int rope_half;         // >0: physical row of logical row p is (p/half)*2*half + p%half
  int vl_len;            // staged vector length per batch row
  int vl_nseg;           // partial sums to add when staging
  int rot;               // rotation of the unit -> CTA assignment (ST_ATTN: item -> warp)
  int cps;               // boxes (column chunks of 512 bytes) per K segment
  int nch;               // SF_Q4: column tiles per tile row, ceil(K / kQ4BoxCols)
  int reserved1;
  int B;                 // batch rows
  int reserved2;         // (explicit padding: programs are compared byte by byte on the host)
  const void* vl_src;    // fp32 (or T with SF_IN_T) [vl_nseg, B, vl_len]
  const void* vl_w;      // RMSNorm weight, type T
  void* out;             // epilogue destination
  const void* resid;     // EPI_RESID addend
  void* cache;           // EPI_ROPE_K / EPI_V: cache base [B, S_max, Hk, Dh] of type T
  const void* cos_tab;   // [S_max, Dh/2] type T
  const void* sin_tab;
  const int* seqlens;    // [B] number of tokens already in the cache (= write position)
  float eps, scale;
  int H, Hk, Dh, S_max;
  // ST_ATTN
  const void* q;         // [B, H*Dh] fp32 (or T with SF_IN_T), already rotated
  const void* kcache;
  const void* vcache;
  float* part_acc;       // [B, H, nsplit, Dh]
  float* part_ml;        // [B, H, nsplit, 2]
  int* counters;         // [B, H] arrival counts of the parts of a head, zero between uses
  int nsplit, seqlen_add;  // keys attended = seqlens[b] + seqlen_add
  // ST_EMBED / ST_ARGMAX
  int* tokens;           // [B] token ids: input of ST_EMBED, output of ST_ARGMAX
  int* token_log;        // [max_steps, B] or null
  int* step_counter;     // incremented once per ST_ARGMAX
  int* seqlens_rw;       // [B] incremented by ST_ARGMAX
  int vocab, max_steps;
  int reserved3[2];
};
static_assert(sizeof(Stage) == 288, "Stage has no implicit padding");

// Persistent words shared by all launches that use one workspace.
struct SyncState {
  unsigned long long arrivals;   // grid-barrier arrival count of the running launch (zero between launches)
  unsigned long long launches;   // launches finished on these words (diagnostics)
  int status;                    // 0 = ok, else first error code raised on the device
  int status_detail;
  unsigned reserved;
  unsigned done_ctas;            // CTAs that have finished the running launch
};

enum DeviceStatus : int {
  DS_OK = 0,
  DS_BARRIER_TIMEOUT = 1,   // a grid-barrier wait ran out
  DS_COPY_TIMEOUT = 2,      // a wait for a ring box ran out
  DS_CACHE_FULL = 4,        // a token arrived at position >= S_max: its key / value were not stored
};

// Geometry of the factor stream.
// 8 warps per CTA: with more, the register file leaves 168 registers per thread and the
// interpreter spills; 256 threads get 255.
constexpr int kConsumerWarps = 7;      // warps that multiply
constexpr int kProducerWarps = 1;      // warp that issues the TMA copies, from one lane per consumer warp
constexpr int kUnitRows = 16;          // factor rows of one unit = rows of one box
// Bytes of one box row.  448 = 7 x 64: consecutive rows start 16 banks apart, so the quarter-warp
// of a 16-byte shared-memory load (two rows x 64 bytes) touches every bank once; with 512 the two
// rows fall on the same 16 banks and every load takes two passes (measured: +14 % tokens/s at
// batch 8, +1.6 % at batch 1).
#ifndef FSVD_BOX_ROW_BYTES
#define FSVD_BOX_ROW_BYTES 448
#endif
constexpr int kBoxRowBytes = FSVD_BOX_ROW_BYTES;
constexpr int kQ4RowBytes = 512;       // bytes of one row of an int4 tile (below)
constexpr int kBoxBytes = kUnitRows * kBoxRowBytes;
constexpr int kMaxSlots = 21;          // ring slots; a multiple of kConsumerWarps

// int4 factors (4-bit codes, symmetric, one fp16 scale per row and group of 128 inputs) are
// stored as a stream of tiles, one tile per box: tile (rt, ct) covers rows [16 rt, 16 rt + 16) and
// inputs [1024 ct, 1024 ct + 1024) and is 17 rows of 512 bytes: rows 0..15 hold the codes of the
// 16 factor rows (eight per 32-bit word: inputs 8 i .. 8 i + 7 in word i, the even ones in the
// nibbles of the low half-word, the odd ones in the high half-word), row 16 holds the 16 x 8 scales
// (fp16, [row][group], 256 bytes) and 256 bytes of zeros.  Codes past the matrix are 8 (= 0 after
// the offset) and scales past it are 0.  Tiles are stored row-major over (rt, ct).
constexpr int kQ4TileRows = kUnitRows + 1;
constexpr int kQ4BoxBytes = kQ4TileRows * kQ4RowBytes;   // 8704
constexpr int kQ4BoxCols = 2 * kQ4RowBytes;              // 1024 inputs per tile
constexpr int kQ4Group = 128;

constexpr int kMaxSmallStages = 14;
struct SmallProgram {
  Stage st[kMaxSmallStages];
};

// 128-byte TMA descriptors of a by-value program, two per stage (operand A, operand B).
struct alignas(64) SmallMaps {
  unsigned char m[2 * kMaxSmallStages][128];
};

// Shared-memory header of the interpreter (two stage descriptors, reduction scratch, the copy
// of a by-value program, the ring's mbarriers), rounded to 1 KB.
constexpr int kStageBytesAl = ((int)sizeof(Stage) + 15) / 16 * 16;
constexpr int kSmallProgBytes = kMaxSmallStages * kStageBytesAl;
FSVD_HD constexpr int smem_header_bytes() {
  return ((2 * kStageBytesAl + 512 + kSmallProgBytes + 512 + 1023) / 1024) * 1024;
}

}  // namespace fsvd
