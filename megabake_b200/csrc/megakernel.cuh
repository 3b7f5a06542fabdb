// Device-side data structures shared by the megakernel and its host launcher.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/megabake_b200.h"

namespace mk {

typedef __nv_bfloat16 bf16;

constexpr int kWorkerWarps = 8;
constexpr int kWorkers = kWorkerWarps * 32;
constexpr int kThreads = 64 + kWorkers + 32;  // warp 0: weight producer, warp 1: MMA issuer, then the workers, last warp: activation producer
constexpr int kTileRows = 128;           // UMMA M; a tile fills only its first `rows` rows
constexpr int kChunkK = 64;              // K elements per weight chunk (128 B of bf16 = one swizzle row)
constexpr int kGranule = 1024;           // weight ring allocation unit (8 rows of 128 B)
constexpr int kRingGranules = 120;       // keeps the CTA under 196 KiB of shared memory so ~60 KiB stay L1 (stack, spills)
constexpr int kRingBytes = kRingGranules * kGranule;
constexpr int kChunkBars = 128;          // full/empty barrier pairs, indexed by chunk sequence number
constexpr int kTok = MK_TOKEN_TILE;      // token columns an epilogue step reads from TMEM
constexpr int kMaxTok = 128;             // largest token tile (UMMA N is 16, 32, 64 or 128)
constexpr int kBSlots = 32;              // activation K-chunks resident per CTA (two halves of 16)
constexpr int kBHalf = kBSlots / 2;
constexpr int kBSlotBytes = kTok * 128;  // 2 KiB
constexpr int kBBytes = kBSlots * kBSlotBytes;
constexpr int kTmemCols = 512;           // 2 buffers x 2 accumulators x 128 columns: all of an SM's tensor memory
constexpr int kMiscBytes = 4096;
constexpr int kMiscTcBytes = 3072;       // tensor engine only: barriers of the activation ring
constexpr int kSmemBytes = 1024 /*alignment slack*/ + kRingBytes + kBBytes + kMiscBytes + kMiscTcBytes;
constexpr int kMaxChunks = 16;           // split-context chunks per (sequence, kv head)
constexpr int kScoreBytes = 40960;       // fp32 scores of one attention unit (inside the B region)
constexpr int kExchangeFloats = 48;      // per (row group, chunk), 192 bytes: max[8], sum[8] as plain floats (the flag protocol) or each
                                         // paired with the phase's stamp in one 64-bit word (16 words), then the two flags
constexpr int kXchStatsFlag = 32;        // float index of "the statistics are out" (flag protocol)
constexpr int kXchPartsFlag = 33;        // float index of "the chunk's partial sums are out"
constexpr int kMaxSplit = 4;             // K slices a projection may be cut into
constexpr int kSplitTokens = 4;          // launches with at most this many tokens use the split-K table

static_assert(kSmemBytes <= 200704, "dynamic shared memory exceeds the 196 KiB carve-out");

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU = 2, EPI_PARTIAL = 3, EPI_ROWRES = 4, EPI_TP = 5 };
enum { B_PLAIN = 0, B_NORM = 1, B_ATTN = 2 };
enum { MODE_DECODE = 0, MODE_PREFILL = 1, MODE_LINEAR = 2, MODE_KVATT = 3, MODE_ATT = 4 };
enum { EV_PHASE_ENTER = 1, EV_B_STAGED = 2, EV_FIRST_ACC = 3, EV_PHASE_DONE = 4, EV_BARRIER_DONE = 5, EV_ATTENTION_DONE = 6,
       EV_ATT_INPUTS = 7, EV_ATT_SCORES = 8, EV_ATT_STATS = 9, EV_ATT_VALUES = 10, EV_ATT_PARTIAL = 11, EV_FIRST_COPY = 12 };
enum {
  SITE_PRODUCER_EMPTY = 1, SITE_MMA_FULL = 2, SITE_MMA_B = 3, SITE_MMA_ACC = 4, SITE_EPI_ACC = 5,
  SITE_GRID_BARRIER = 6, SITE_ATT_EXCHANGE = 7, SITE_DRAIN = 8, SITE_PROLOGUE = 9, SITE_B_EMPTY = 10,
  SITE_TP_FLAG = 11, SITE_KV_TILE = 12
};
constexpr int kMaxTp = 8;                // ranks of a tensor-parallel group (one node, NVLink peers)
constexpr int kTpFlagBytes = 256;        // head of a rank's exchange buffer: one arrival stamp per peer

// One projection phase: up to three weight matrices sharing the same activation
// operand (q,k,v), or a gate/up pair accumulated side by side (nacc == 2).
// Output rows are cut into tiles of `rows` rows (<= 128) and the reduction
// length into `ksplit` slices; a unit is (row tile, K slice).  rows and ksplit
// are chosen on the host so that the unit count is just under a multiple of the
// CTA count and a TMA box (rows x 128 B) stays large; CTA c takes units c,
// c+grid, ...  With ksplit == 1 a unit finishes its outputs in one fp32 chain.
// With ksplit > 1 (EPI_PARTIAL) each unit stores fp32 partial sums and the next
// phase adds them, in slice order, while it builds its activation operand.
struct GemmPhase {
  const CUtensorMap* tmap[3];  // device copies of the weights' TMA descriptors (tensor engine: box = 64 x rows x kb chunks)
  const CUtensorMap* bmap[4];  // tensor engine: descriptors of the token operand for token tiles of 16, 32, 64, 128 (box = 64 x tile)
  const bf16* w[3];            // raw weight pointers [N, K]
  const bf16* bias[3];
  int n[3];                    // rows of each matrix
  int tile_start[4];           // first row tile of each matrix, then the total
  int out_col[3];              // column of each matrix's rows in the output buffer
  int nseg, nacc;
  int k, kc;                   // reduction length, in elements and in 64-element chunks
  int rows;                    // weight rows per tile
  int kb;                      // K chunks one weight copy brings (tensor engine: kb swizzled chunks of rows x 128 B per matrix;
                               // small-launch kernel: unswizzled boxes of kb * 64 elements x rows)
  int gran;                    // ring granules one entry occupies (tensor engine: nacc * kb * rows / 8)
  int gate;                    // tensor engine: 1 = this phase follows decode attention, whose cache tiles stream through the weight
                               // ring: its weights may be fetched only once the workers have released the ring (a_ready)
  int map3d;                   // tensor engine: 1 = tmap is three-dimensional and one copy brings kb chunks; 0 = one 2-D copy per chunk
  int ntiles;                  // row tiles
  int ksplit, kslice;          // K slices and chunks per slice (kc == ksplit * kslice)
  int nunits;                  // ntiles * ksplit
  int epi, bmode;
  int gather;                  // 1: activation rows are embedding rows selected by the token ids
  int to_logits;               // 1: output goes to the caller's logits buffer
  int ll;                      // small-launch table: 1 = the bf16 outputs of this phase leave as 64-bit words
                               // {stamp, bf16 pair} in ll_dst, which the consumer polls instead of waiting at a grid barrier
  int ll_ld, ll_src_ld;        // words per token in ll_dst / ll_src
  unsigned long long* ll_dst;
  const unsigned long long* ll_src;  // B_PLAIN / B_NORM: the operand as stamped bf16 pairs; B_ATTN: attention partials as {stamp, fp32}
  int bulk;                    // one-token row table: 1 = a tile is `rows` whole weight rows, contiguous in memory, fetched by
  int rpc;                     // one-dimensional bulk copies of `rpc` rows; the epilogue (EPI_ROWRES) adds the residual it
  const unsigned long long* res_src;  // reads as stamped pairs from res_src (or the embedding row when `gather`) and stamps the sum into ll_dst
  int tp_buf;                  // EPI_TP: which half of the exchange buffers this projection's partial sums go to
  int add_parts;               // B_NORM: fp32 partial slices of the previous projection to add to the residual
  const bf16* normw;
  const bf16* src; int src_ld; // activation source (B_NORM: the residual stream before this phase)
  bf16* dst; int dst_ld;
  float* partial;              // EPI_PARTIAL output / B_NORM add_parts input: [slice][token][hidden]
  bf16* h_out;                 // B_NORM with add_parts or gather: where the updated residual stream goes
};

struct Control {
  uint32_t barrier;   // monotonic grid-barrier counter
  uint32_t abort;     // set once by whoever gives up a wait; every wait polls it
  int status;         // mk_device_status
  int where, cta, detail;
  int att_nch;        // context chunks the last attention phase used (read by the o projection)
  uint32_t pad;
};

struct KParams {
  int hidden, layers, q_heads, kv_heads, head_dim, inter, vocab;
  int embed_rows;     // rows of the embedding table (token ids are checked against it); vocab = rows of this rank's lm_head
  float eps;
  int rope_style, prefill_rope_style;
  float att_scale;    // head_dim ** -0.5 rounded to fp32 on the host
  int mode;
  int m;              // tokens in this launch
  int batch, seq;
  int capacity;
  int engine;
  int n_gemm;         // projection phases in this launch
  int nbar;           // grid barriers a CTA passes in this launch
  uint32_t epoch;     // barrier counter value when this launch starts
  uint32_t att_epoch; // attention phases run before this launch (exchange stamps count up from it)
  int qkv_ld;
  int max_positions;
  int stream_once;    // 1: weights are read once per launch (L2 evict-first)
  int split;          // 1: this launch runs the split-K phase table (residual updates applied by the consumer)
  int rowmode;        // 1: one-token row table: stamped hand-offs everywhere, one grid barrier at the end of the launch
  int ragged;         // 1: len[l] points to one valid length per sequence (int32 [batch]) instead of one shared by the batch
  int sample;         // 1: after the logits, pick each sequence's greedy token on the device, store it in tokens_out and as the
                      //    next id, and advance the position: the next launch needs no host round trip
  long long* tokens_out;      // [m] with `sample`
  volatile int* status_mirror;  // host-mapped copy of Control::status (pinned memory), or null
  int trace_cap;      // events per CTA in `trace` (0 = tracing off)
  unsigned long long* trace;  // [grid][trace_cap] (event code << 56) | %globaltimer ns
  long long timeout_cycles;
  const GemmPhase* phases;
  bf16 *hidden_buf, *qkv, *attn, *act;
  bf16* xnorm;        // [m][hidden]: the normalised rows a norm phase leaves for the projections that follow
  unsigned long long* qkv_ll;  // [kSplitTokens][qkv width / 2]: stamped q/k/v outputs of the small-launch kernel
  unsigned long long* att_ll;  // [kSplitTokens * q_heads][kMaxChunks][head_dim]: stamped attention partials {stamp, fp32}
  unsigned long long* attn_ll; // [kSplitTokens][q_heads * head_dim / 2]: the combined attention output as stamped bf16 pairs
  float* att_xch;     // [row groups][kMaxChunks][kExchangeFloats]
  float* att_part;    // [batch * q_heads][kMaxChunks][head_dim]
  Control* ctrl;
  long long* ids;     // read by every CTA; rewritten at the very end of a launch with `sample`
  long long* pos;
  // Tensor parallel group (tp_size > 1): this rank holds q_heads, kv_heads and inter of its shard; o_proj and
  // down_proj produce partial sums over the rank's share of the reduction length.  tp_peer[r] is rank r's
  // exchange buffer as this process addresses it (peer-mapped; tp_peer[tp_rank] is local):
  //   [kTpFlagBytes: uint32 stamp per source rank][2 halves][tp_size source ranks][m tokens][hidden] fp32
  int tp_rank, tp_size;
  uint32_t tp_epoch;  // all-reduces this group has finished before this launch (stamps count up from it)
  uint8_t* tp_peer[kMaxTp];
  const bf16* mask;
  const bf16 *embed, *cos_t, *sin_t;
  bf16* logits;
  // stand-alone attention ops
  const bf16 *op_q, *op_k, *op_v;
  bf16* op_out;
  int op_qlen, op_klen;
  // stand-alone projection (MODE_LINEAR): its phase and its two descriptors travel in the parameter block,
  // so the call needs no upload and no synchronisation
  GemmPhase linear_phase;
  int small_ring;  // weight ring of the small-launch kernel, in 1 KiB granules
  const CUtensorMap* kv_maps;  // decode on the tensor engine: 4-D descriptors of the key caches [layers], then of the value caches [layers]; null = plain copies
  CUtensorMap linear_wmap, linear_xmap;
  void* kc[MK_MAX_LAYERS];
  void* vc[MK_MAX_LAYERS];
  int* len[MK_MAX_LAYERS];
};

static_assert(sizeof(KParams) <= 4096, "the parameter block must stay within the classic 4 KB kernel-parameter limit");

}  // namespace mk
