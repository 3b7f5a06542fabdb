// Host side of the C ABI declared in include/megabake_b200.h: workspace carving,
// TMA descriptor encoding, the per-launch parameter block and the cooperative
// launch of the megakernel.  No device memory is allocated here.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <algorithm>
#include <vector>

#include "decode_small.cuh"

using namespace mk;

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

#define MK_CUDA(call)                                                                       \
  do {                                                                                      \
    cudaError_t e_ = (call);                                                                \
    if (e_ != cudaSuccess) return fail(MK_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Carve {
  size_t ctrl, tmaps, kvmaps, phases, hidden, hidden2, xnorm, qkv, qkv_ll, act_ll, att_ll, attn_ll, res_a, res_b, attn, act, partial, partial2, att_xch, att_part, host_io, total;
};

int qkv_width(const mk_config& c) { return (c.q_heads + 2 * c.kv_heads) * c.head_dim; }
// Token-operand descriptors of the tensor engine: (normalised rows, attention output, SiLU*up, mk_linear's
// source) x (token tiles of 16, 32, 64), behind the weight descriptors.
constexpr int kCacheMapSets = 8;  // cache-descriptor sets a handle remembers (one per KV state it is called with in turn)
constexpr int kOperandTiles = 4;  // token tiles of 16, 32, 64, 128
constexpr int kOperandKinds = 4, kOperandMaps = kOperandKinds * kOperandTiles;
enum { OPERAND_XNORM = 0, OPERAND_ATTN = 1, OPERAND_ACT = 2, OPERAND_LINEAR = 3 };
int token_tile_of(int m) { return m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128)); }
size_t maps_per_table(const mk_config& c) { return 7 * static_cast<size_t>(c.layers) + 1; }
size_t phases_per_table(const mk_config& c) { return 4 * static_cast<size_t>(c.layers) + 1; }

Carve carve(const mk_config& c) {
  Carve v{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align_up(off + bytes, 256);
    return at;
  };
  const size_t m = static_cast<size_t>(c.max_tokens);
  v.ctrl = take(sizeof(Control));
  v.tmaps = take(sizeof(CUtensorMap) * (4 * maps_per_table(c) + 1 + kOperandMaps));  // split, plain and small-launch tables, mk_linear, token operands, row table
  v.kvmaps = take(sizeof(CUtensorMap) * 2 * static_cast<size_t>(c.layers) * kCacheMapSets);  // decode attention: per set, key caches then value caches
  v.phases = take(sizeof(GemmPhase) * (4 * phases_per_table(c) + 1));  // + the one-token row table
  v.hidden = take(m * c.hidden * 2);
  v.hidden2 = take(m * c.hidden * 2);
  v.xnorm = take(m * c.hidden * 2);
  v.qkv = take(m * qkv_width(c) * 2);
  v.qkv_ll = take(static_cast<size_t>(kSplitTokens) * qkv_width(c) * 4);
  v.act_ll = take(static_cast<size_t>(kSplitTokens) * c.intermediate * 4);
  v.att_ll = take(static_cast<size_t>(kSplitTokens) * c.q_heads * kMaxChunks * c.head_dim * 8);
  v.attn_ll = take(static_cast<size_t>(kSplitTokens) * c.q_heads * c.head_dim * 4);
  v.res_a = take(static_cast<size_t>(kSplitTokens) * c.hidden * 4);  // stamped residual stream after the MLP
  v.res_b = take(static_cast<size_t>(kSplitTokens) * c.hidden * 4);  // ... and after attention
  v.attn = take(m * c.q_heads * c.head_dim * 2);
  v.act = take(m * c.intermediate * 2);
  v.partial = take(static_cast<size_t>(kMaxSplit) * std::max<size_t>(m, kSplitTokens) * c.hidden * 4);
  v.partial2 = take(static_cast<size_t>(kMaxSplit) * kSplitTokens * c.hidden * 4);  // down-proj partials of the small-launch table
  v.att_xch = take(m * c.kv_heads * kMaxChunks * kExchangeFloats * 4);
  v.att_part = take(m * c.q_heads * kMaxChunks * c.head_dim * 4);
  v.host_io = take(3 * m * sizeof(int64_t));  // mk_decode_step_host: ids, positions, sampled tokens
  v.total = off;
  return v;
}

int check_config(const mk_config& c) {
  if (c.hidden <= 0 || c.layers <= 0 || c.q_heads <= 0 || c.kv_heads <= 0 || c.intermediate <= 0 || c.vocab <= 0 ||
      c.max_tokens <= 0 || c.max_positions <= 0)
    return fail(MK_ERR_INVALID, "config: every size must be positive");
  if (c.layers > MK_MAX_LAYERS) return fail(MK_ERR_UNSUPPORTED, "config: at most %d layers", MK_MAX_LAYERS);
  if (c.head_dim != 64 && c.head_dim != 128) return fail(MK_ERR_UNSUPPORTED, "config: head_dim must be 64 or 128");
  if (c.q_heads % c.kv_heads) return fail(MK_ERR_INVALID, "config: q_heads must be a multiple of kv_heads");
  if (c.q_heads / c.kv_heads > 8) return fail(MK_ERR_UNSUPPORTED, "config: at most 8 query heads per kv head");
  if (c.hidden % 64 || c.intermediate % 64)
    return fail(MK_ERR_UNSUPPORTED, "config: hidden and intermediate must be multiples of 64");
  if (c.hidden > kNormVecs * kWorkers * 8)
    return fail(MK_ERR_UNSUPPORTED, "config: hidden above %d (a norm phase keeps a row in the registers of one CTA)", kNormVecs * kWorkers * 8);
  if (c.engine != MK_ENGINE_TCGEN05 && c.engine != MK_ENGINE_FMA && c.engine != MK_ENGINE_AUTO)
    return fail(MK_ERR_INVALID, "config: engine");
  if (c.rope_style != MK_ROPE_HF && c.rope_style != MK_ROPE_HALF_SWAP) return fail(MK_ERR_INVALID, "config: rope_style");
  if (c.tp_size < 0 || c.tp_size > kMaxTp) return fail(MK_ERR_UNSUPPORTED, "config: tensor-parallel groups have 1..%d ranks", kMaxTp);
  if (c.tp_size > 1 && (c.tp_rank < 0 || c.tp_rank >= c.tp_size)) return fail(MK_ERR_INVALID, "config: tp_rank outside the group");
  if (c.embed_rows < 0) return fail(MK_ERR_INVALID, "config: embed_rows");
  return MK_OK;
}

int device_grid(const mk_config& c, int device, int* grid) {
  int sms = 0;
  MK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  *grid = (c.sm_limit > 0 && c.sm_limit < sms) ? c.sm_limit : sms;
  return MK_OK;
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
  });
  return fn;
}

// bf16 [rows, k] row-major -> boxes of box_rows rows x 64 columns, 128-byte swizzle.
int encode_weight_map(CUtensorMap* out, const void* base, int rows, int k, int box_rows, int box_chunks = 1,
                      bool swizzle = true) {
  if (reinterpret_cast<uintptr_t>(base) % 16) return fail(MK_ERR_ALIGNMENT, "weight base %p is not 16-byte aligned", base);
  auto fn = encode_fn();
  if (!fn) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  // swizzle: the tensor core's operand layout (64 elements = 128 bytes per row, 128-byte swizzle).
  // !swizzle: plain rows of box_chunks * 128 bytes for the CUDA-core consumer (up to 256 elements).
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kChunkK * box_chunks), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (rows %d, k %d)", (int)r, rows, k);
  return MK_OK;
}

// Tensor engine, weights: bf16 [rows, k] row-major seen as (64 elements, rows, k / 64 chunks); a box is
// box_rows rows x box_chunks chunks, each chunk 128-byte swizzled: one copy brings several K chunks of a tile.
int encode_weight_map3(CUtensorMap* out, const void* base, int rows, int k, int box_rows, int box_chunks) {
  if (reinterpret_cast<uintptr_t>(base) % 16) return fail(MK_ERR_ALIGNMENT, "weight base %p is not 16-byte aligned", base);
  auto fn = encode_fn();
  if (!fn) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kChunkK), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(k / kChunkK)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k) * 2, static_cast<cuuint64_t>(kChunkK) * 2};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(kChunkK), static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(box_chunks)};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with %d (rows %d, k %d, box %d x %d)", (int)r, rows, k, box_rows, box_chunks);
  return MK_OK;
}

// The weight descriptor of a tensor-engine phase: three-dimensional when the driver accepts the chunk-major
// view (its chunk stride, 128 bytes, is smaller than its row stride), else one 64-column box per copy.
int encode_phase_weight_map(CUtensorMap* out, const void* base, int rows, int k, GemmPhase& ph, bool& use3d) {
  if (use3d) {
    if (encode_weight_map3(out, base, rows, k, ph.rows, ph.kb) == MK_OK) {
      ph.map3d = 1;
      return MK_OK;
    }
    use3d = false;  // fall back for this and every later matrix of the handle
  }
  ph.map3d = 0;
  return encode_weight_map(out, base, rows, k, ph.rows);
}

// Tensor engine, token operand: bf16 [tokens, k] row-major, box = 64 elements x `tile` tokens, 128-byte
// swizzle; token rows past `tokens` read as zeros.
int encode_operand_map(CUtensorMap* out, const void* base, int tokens, int k, int tile) {
  if (reinterpret_cast<uintptr_t>(base) % 16) return fail(MK_ERR_ALIGNMENT, "operand base %p is not 16-byte aligned", base);
  auto fn = encode_fn();
  if (!fn) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kChunkK), static_cast<cuuint32_t>(tile)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled (operand) failed with %d (tokens %d, k %d)", (int)r, tokens, k);
  return MK_OK;
}

// Decode attention on the tensor engine: a cache [batch, capacity, kv_heads * head_dim] seen as
// (64 dimensions, positions, 64-dimension chunks of a row, sequences); a box is one stage of a unit:
// 64 x tile_keys positions x the unit's chunks, each chunk 128-byte swizzled.
int encode_cache_map(CUtensorMap* out, const void* base, int batch, int capacity, int row_elems, int tile_keys, int unit_chunks) {
  if (reinterpret_cast<uintptr_t>(base) % 16) return fail(MK_ERR_ALIGNMENT, "cache base %p is not 16-byte aligned", base);
  auto fn = encode_fn();
  if (!fn) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(kChunkK), static_cast<cuuint64_t>(capacity),
                              static_cast<cuuint64_t>(row_elems / kChunkK), static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(row_elems) * 2, static_cast<cuuint64_t>(kChunkK) * 2,
                                 static_cast<cuuint64_t>(capacity) * row_elems * 2};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(kChunkK), static_cast<cuuint32_t>(tile_keys), static_cast<cuuint32_t>(unit_chunks), 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MK_ERR_CUDA, "cuTensorMapEncodeTiled (cache) failed with %d", (int)r);
  return MK_OK;
}

}  // namespace

struct mk_handle_s {
  mk_config cfg;
  int device, grid;
  uint8_t* ws;
  Carve cv;
  bool bound;
  mk_weights weights;
  std::vector<mk_layer_weights> layers;
  uint32_t epoch, att_epoch;
  int64_t launches;
  long long timeout_cycles;
  float att_scale;
  bool fma_ok;  // the small-launch kernel can run the split-K table: every K slice fits its fp32 operand buffer
  bool row_ok;    // the one-token row table (no K split, no per-layer grid barrier) is available
  bool small_ll;  // its q/k/v phases hand their outputs to attention as stamped words (one grid barrier fewer per layer)
  unsigned long long* trace;
  int trace_cap;
  int small_ring;       // weight ring of the small-launch kernel, 1 KiB granules
  int fat_copy;         // largest weight copy of the small-launch tables, bytes (three to four fit the ring)
  struct CacheMapSet {
    std::vector<const void*> seen;  // cache pointers the set's descriptors were encoded for (keys, then values)
    int capacity = 0, batch = 0;
    uint64_t used = 0;              // launch counter at the last use (least recently used is replaced)
  };
  CacheMapSet kv_sets[kCacheMapSets];
  bool kv_maps_ok;      // the driver takes the four-dimensional view of a cache
  bool use3d;           // weight descriptors of the tensor engine are three-dimensional (several K chunks per copy)
  uint32_t tp_epoch;    // all-reduces launched so far (tensor parallel)
  uint8_t* tp_peer[kMaxTp];
  bool tp_bound;
  volatile int* mirror;  // host-mapped status word, or null
  std::mutex lock;
};

namespace {

template <typename T>
T* at(mk_handle h, size_t off) { return reinterpret_cast<T*>(h->ws + off); }

// Rows per tile: the smallest height for which the phase's row tiles fit in the
// fewest possible rounds over `slots` CTAs (each round gives every CTA one unit).
int choose_rows(const GemmPhase& ph, int slots, int max_rows = kTileRows) {
  const int nseg = ph.nacc == 2 ? 1 : ph.nseg;
  long long total = 0;
  for (int s = 0; s < nseg; ++s) total += ph.n[s];
  if (slots < 1) slots = 1;
  for (long long rounds = (total + static_cast<long long>(max_rows) * slots - 1) / (static_cast<long long>(max_rows) * slots);;
       ++rounds) {
    for (int rows = static_cast<int>((total + rounds * slots - 1) / (rounds * slots)); rows <= max_rows; ++rows) {
      long long tiles = 0;
      for (int s = 0; s < nseg; ++s) tiles += (ph.n[s] + rows - 1) / rows;
      if (tiles <= rounds * slots) return rows;
    }
  }
}

// A TMA box of fewer than ~40 rows (5 KB) cannot keep an SM's share of HBM
// bandwidth busy (the copy engine retires roughly one box per 0.1 us), so a
// projection with few output rows per CTA is cut along K as well.
constexpr int kGoodBoxRows = 40;

void finish_phase(GemmPhase& ph, int grid, bool allow_split, int max_rows = kTileRows) {
  ph.kc = ph.k / kChunkK;
  int best_split = 1, best_rows = choose_rows(ph, grid, max_rows);
  if (allow_split && best_rows < kGoodBoxRows) {
    static const int candidates[] = {2, 3, 4};
    for (int split : candidates) {
      if (ph.kc % split || ph.kc / split < 2 || grid / split < 1) continue;
      const int rows = choose_rows(ph, grid / split, max_rows);
      if (rows > best_rows) {
        best_rows = rows;
        best_split = split;
      }
      if (rows >= kGoodBoxRows) break;
    }
  }
  ph.ksplit = best_split;
  ph.kslice = ph.kc / best_split;
  ph.rows = best_rows;
  ph.kb = 1;
  ph.gran = (ph.rows * 128 + kGranule - 1) / kGranule;
  const int nseg = ph.nacc == 2 ? 1 : ph.nseg;
  int tile = 0;
  for (int s = 0; s < nseg; ++s) {
    ph.tile_start[s] = tile;
    tile += (ph.n[s] + ph.rows - 1) / ph.rows;
  }
  ph.tile_start[nseg] = tile;
  ph.ntiles = tile;
  ph.nunits = tile * best_split;
}

// Tensor engine: tile heights are multiples of 8 (a swizzled chunk of a tile must start on a 1 KiB boundary
// inside a ring entry), and an entry carries `kb` K chunks per matrix: as many as divide the K range and keep
// the entry under ~36 KB (three entries of the 120 KB ring in flight); two at most when launches can have
// token tiles of 64 (the activation ring holds 64 KB).
void finish_phase_tc(GemmPhase& ph, int grid, bool allow_split, int max_tokens) {
  finish_phase(ph, grid, allow_split);
  ph.rows = std::min(kTileRows, (ph.rows + 7) / 8 * 8);
  const int nseg = ph.nacc == 2 ? 1 : ph.nseg;
  int tile = 0;
  for (int s = 0; s < nseg; ++s) {
    ph.tile_start[s] = tile;
    tile += (ph.n[s] + ph.rows - 1) / ph.rows;
  }
  ph.tile_start[nseg] = tile;
  ph.ntiles = tile;
  ph.nunits = tile * ph.ksplit;
  int kb = 1;
  for (int cand = 2; cand <= (max_tokens > 32 ? 2 : 4); ++cand)
    if (ph.kslice % cand == 0 && ph.nacc * cand * ph.rows * 128 <= 36 * 1024) kb = cand;
  ph.kb = kb;
  ph.gran = ph.nacc * kb * ph.rows / 8;
}

// The split-K table (o_proj and down_proj cut along K so that every SM streams, fp32 partial sums added by
// the next norm phase) serves every launch of a single-GPU handle.  The small-launch kernel further needs a
// reduction length of at most 2048 per K slice (its fp32 operand buffer).
bool split_table_ok(const mk_config& c) { return c.tp_size <= 1; }
bool small_shape_ok(const mk_config& c) { return c.hidden / kChunkK <= kBSlots && c.tp_size <= 1; }

// One-token launches run the row table with the handle's ring; the split-K table of two to four tokens
// measured best with a 92 KiB ring and copies of at most 30 KiB.
constexpr int kSplitTableRing = 92;
constexpr int kBoxCopyBytes = 30 * 1024;
int small_ring_for(mk_handle h, int tokens) { return tokens == 1 ? h->small_ring : std::min(h->small_ring, kSplitTableRing); }

void base_params(mk_handle h, KParams& p) {
  memset(&p, 0, sizeof(p));
  const mk_config& c = h->cfg;
  p.hidden = c.hidden; p.layers = c.layers; p.q_heads = c.q_heads; p.kv_heads = c.kv_heads;
  p.head_dim = c.head_dim; p.inter = c.intermediate; p.vocab = c.vocab; p.eps = c.rms_eps;
  p.embed_rows = c.embed_rows > 0 ? c.embed_rows : c.vocab;
  p.tp_size = c.tp_size > 1 ? c.tp_size : 1;
  p.tp_rank = c.tp_size > 1 ? c.tp_rank : 0;
  p.tp_epoch = h->tp_epoch;
  for (int r = 0; r < kMaxTp; ++r) p.tp_peer[r] = h->tp_peer[r];
  p.rope_style = c.rope_style; p.prefill_rope_style = MK_ROPE_HF;
  p.att_scale = h->att_scale;
  p.engine = MK_ENGINE_TCGEN05;
  p.epoch = h->epoch;
  p.att_epoch = h->att_epoch;
  p.qkv_ld = qkv_width(c);
  p.max_positions = c.max_positions;
  p.timeout_cycles = h->timeout_cycles;
  p.trace = h->trace;
  p.trace_cap = h->trace ? h->trace_cap : 0;
  p.status_mirror = h->mirror;
  p.small_ring = small_ring_for(h, 1);  // launches of two to four tokens overwrite it
  p.ctrl = at<Control>(h, h->cv.ctrl);
  p.att_xch = at<float>(h, h->cv.att_xch);
  p.att_part = at<float>(h, h->cv.att_part);
  if (h->cv.phases == 0) return;  // a view without decoder buffers (the static-scratch attention): the rest stays null
  p.phases = at<GemmPhase>(h, h->cv.phases);
  p.hidden_buf = at<bf16>(h, h->cv.hidden);
  p.xnorm = at<bf16>(h, h->cv.xnorm);
  p.qkv = at<bf16>(h, h->cv.qkv);
  p.attn = at<bf16>(h, h->cv.attn);
  p.act = at<bf16>(h, h->cv.act);
  p.qkv_ll = at<unsigned long long>(h, h->cv.qkv_ll);
  p.att_ll = at<unsigned long long>(h, h->cv.att_ll);
  p.attn_ll = at<unsigned long long>(h, h->cv.attn_ll);
  p.embed = static_cast<const bf16*>(h->weights.embed);
  p.cos_t = static_cast<const bf16*>(h->weights.rope_cos);
  p.sin_t = static_cast<const bf16*>(h->weights.rope_sin);
}

// The small-launch kernel is instantiated per token count (1..kSplitTokens).
// One kernel per token count, and one more for the one-token row table (`row`): code that is compiled in
// but never runs still costs instruction-cache reach.
const void* small_kernel(int tokens, bool row) {
  if (row) return reinterpret_cast<const void*>(&megakernel_small<1, true>);
  switch (tokens) {
    case 1: return reinterpret_cast<const void*>(&megakernel_small<1, false>);
    case 2: return reinterpret_cast<const void*>(&megakernel_small<2, false>);
    case 3: return reinterpret_cast<const void*>(&megakernel_small<3, false>);
    default: return reinterpret_cast<const void*>(&megakernel_small<4, false>);
  }
}

int prepare_small_kernels(int device, int ring_granules) {
  for (int t = 0; t <= kSplitTokens; ++t) {  // 0: the row-table kernel
    const void* fn = small_kernel(t, t == 0);
    const int bytes = small_smem_bytes(t == 0 ? ring_granules : std::min(ring_granules, kSplitTableRing));
    MK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    MK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, (bytes * 100 + 233471) / 233472));
    int per_sm = 0;
    MK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kSmallThreads, bytes));
    if (per_sm < 1) return fail(MK_ERR_UNSUPPORTED, "the small-launch megakernel does not fit on an SM of device %d", device);
  }
  return MK_OK;
}

int launch(mk_handle h, KParams& p, void* stream, int attention_phases = 0, bool small = false) {
  void* args[] = {&p};
  if (small)
    MK_CUDA(cudaLaunchCooperativeKernel(small_kernel(p.m, p.rowmode != 0), dim3(h->grid), dim3(kSmallThreads), args, small_smem_bytes(p.small_ring),
                                        static_cast<cudaStream_t>(stream)));
  else
    MK_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(&megakernel), dim3(h->grid), dim3(kThreads), args,
                                        kSmemBytes, static_cast<cudaStream_t>(stream)));
  h->epoch += static_cast<uint32_t>(p.nbar) * static_cast<uint32_t>(h->grid);
  h->att_epoch += static_cast<uint32_t>(attention_phases);
  h->launches += 1;
  return MK_OK;
}

int token_tiles(int m) { return (m + token_tile_of(m) - 1) / token_tile_of(m); }

int attention_fits(mk_handle h, int keys, const char* what) {
  const int gs = h->cfg.q_heads / h->cfg.kv_heads;
  const int heads = gs * decode_heads_per_unit(h->cfg.kv_heads, gs, h->cfg.head_dim);  // query heads of one attention unit
  const int max_len = (kScoreBytes / 4 / heads) & ~7;
  const int need = (keys + max_len - 1) / max_len;
  if (need > kMaxChunks || need > h->grid)
    return fail(MK_ERR_UNSUPPORTED, "%s: %d keys exceed %d chunks of %d", what, keys, kMaxChunks, max_len);
  return MK_OK;
}

}  // namespace

extern "C" {

const char* mk_last_error(void) { return g_error; }

size_t mk_workspace_bytes(const mk_config* config, int device) {
  if (!config || check_config(*config) != MK_OK) return 0;
  int grid = 0;
  if (device_grid(*config, device, &grid) != MK_OK) return 0;
  return carve(*config).total;
}

int mk_create(const mk_config* config, void* workspace, size_t workspace_bytes, int device, void* stream,
              mk_handle* out) {
  if (!config || !workspace || !out) return fail(MK_ERR_INVALID, "mk_create: null argument");
  if (int e = check_config(*config)) return e;
  if (reinterpret_cast<uintptr_t>(workspace) % 256) return fail(MK_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  MK_CUDA(cudaSetDevice(device));
  int grid = 0;
  if (int e = device_grid(*config, device, &grid)) return e;
  const Carve cv = carve(*config);
  if (workspace_bytes < cv.total)
    return fail(MK_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", workspace_bytes, cv.total);
  int major = 0, coop = 0, khz = 0;
  MK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  MK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
  MK_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device));
  if (major != 10) return fail(MK_ERR_UNSUPPORTED, "device %d is sm_%d0; this library is built for sm_100a only", device, major);
  if (!coop) return fail(MK_ERR_UNSUPPORTED, "device %d does not support cooperative launch", device);
  MK_CUDA(cudaFuncSetAttribute(megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  MK_CUDA(cudaFuncSetAttribute(megakernel, cudaFuncAttributePreferredSharedMemoryCarveout, (kSmemBytes * 100 + 233471) / 233472));
  int per_sm = 0;
  MK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, megakernel, kThreads, kSmemBytes));
  if (per_sm < 1) return fail(MK_ERR_UNSUPPORTED, "the megakernel does not fit on an SM of device %d", device);
  // Tunables of the small-launch kernel (process-wide: shared-memory attributes belong to the function).
  int small_ring = kSmallRingGranules, fat_copy = 36 * 1024;
  if (const char* env = getenv("MEGABAKE_SMALL_RING_KB")) small_ring = std::max(64, std::min(kSmallRingMax, atoi(env)));
  if (const char* env = getenv("MEGABAKE_SMALL_COPY_KB")) fat_copy = std::max(16, std::min(small_ring / 2, atoi(env))) * 1024;
  if (int e = prepare_small_kernels(device, small_ring)) return e;
  mk_handle h = new (std::nothrow) mk_handle_s();
  if (!h) return fail(MK_ERR_INVALID, "out of host memory");
  h->small_ring = small_ring;
  h->fat_copy = fat_copy;
  h->cfg = *config;
  h->device = device;
  h->grid = grid;
  h->ws = static_cast<uint8_t*>(workspace);
  h->cv = cv;
  h->bound = false;
  h->epoch = 0;
  h->att_epoch = 0;
  h->launches = 0;
  h->trace = nullptr;
  h->trace_cap = 0;
  h->mirror = nullptr;
  {  // does this driver take the chunk-major three-dimensional view of a weight matrix?
    CUtensorMap probe;
    h->use3d = getenv("MEGABAKE_NO_3D_MAPS") == nullptr &&
               encode_weight_map3(&probe, workspace, 128, 256, 64, 2) == MK_OK;
  }
  h->kv_maps_ok = getenv("MEGABAKE_NO_CACHE_MAPS") == nullptr;
  h->tp_epoch = 0;
  h->tp_bound = false;
  for (int r = 0; r < kMaxTp; ++r) h->tp_peer[r] = nullptr;
  double ms = 2000.0;
  if (const char* env = getenv("MEGABAKE_WAIT_LIMIT_MS")) ms = atof(env) > 0 ? atof(env) : ms;
  h->timeout_cycles = static_cast<long long>(ms * static_cast<double>(khz));
  h->att_scale = static_cast<float>(std::pow(static_cast<double>(config->head_dim), -0.5));
  memset(&h->weights, 0, sizeof(h->weights));
  cudaError_t e = cudaMemsetAsync(workspace, 0, cv.total, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    delete h;
    return fail(MK_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  }
  *out = h;
  return MK_OK;
}

int mk_destroy(mk_handle h) {
  delete h;
  return MK_OK;
}

int mk_bind_weights(mk_handle h, const mk_weights* w, void* stream) {
  if (!h || !w || !w->layers) return fail(MK_ERR_INVALID, "mk_bind_weights: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  const mk_config& c = h->cfg;
  if (!w->embed || !w->final_norm || !w->lm_head || !w->rope_cos || !w->rope_sin)
    return fail(MK_ERR_INVALID, "mk_bind_weights: embed, final_norm, lm_head and the rope tables are required");
  const int L = c.layers;
  const int q_size = c.q_heads * c.head_dim, kv_size = c.kv_heads * c.head_dim;
  const size_t nmaps = maps_per_table(c), nphases = phases_per_table(c);
  std::vector<CUtensorMap> maps(3 * nmaps);
  std::vector<GemmPhase> phases(4 * nphases);
  CUtensorMap* dmaps = at<CUtensorMap>(h, h->cv.tmaps);
  CUtensorMap* operand_maps = dmaps + 3 * nmaps + 1;
  CUtensorMap* row_dmaps = operand_maps + kOperandMaps;  // the one-token row table's own (plain-row) descriptors
  std::vector<CUtensorMap> row_maps(nmaps);
  bf16* hidden_a = at<bf16>(h, h->cv.hidden);
  bf16* hidden_b = at<bf16>(h, h->cv.hidden2);
  bf16* qkv = at<bf16>(h, h->cv.qkv);
  bf16* attn = at<bf16>(h, h->cv.attn);
  bf16* act = at<bf16>(h, h->cv.act);
  float* partial = at<float>(h, h->cv.partial);
  for (int l = 0; l < L; ++l) {
    const mk_layer_weights& lw = w->layers[l];
    if (!lw.input_norm || !lw.q || !lw.k || !lw.v || !lw.o || !lw.post_norm || !lw.gate || !lw.up || !lw.down)
      return fail(MK_ERR_INVALID, "mk_bind_weights: layer %d has a null weight", l);
    if (c.qkv_bias && (!lw.q_bias || !lw.k_bias || !lw.v_bias))
      return fail(MK_ERR_INVALID, "mk_bind_weights: layer %d lacks a q/k/v bias", l);
  }
  // Table 0: split-K (small launches): o and down store K-slice partials; the next
  // normalising phase adds them to the residual stream, which ping-pongs between
  // hidden_b (after attention) and hidden_a (after the MLP).  Table 1: plain.
  bool use3d = h->use3d;
  for (int table = 0; table < 2; ++table) {
    const bool split = (table == 0);
    if (split && !split_table_ok(c)) continue;
    GemmPhase* tp = phases.data() + table * nphases;
    CUtensorMap* tmaps_host = maps.data() + table * nmaps;
    CUtensorMap* tmaps_dev = dmaps + table * nmaps;
    int prev_parts = 0;  // K slices of the projection whose partials the next normalising phase adds
    for (int l = 0; l < L; ++l) {
      const mk_layer_weights& lw = w->layers[l];
      GemmPhase* ph = tp + 4 * l;
      memset(ph, 0, sizeof(GemmPhase) * 4);
      // q, k, v
      ph[0].nseg = 3; ph[0].nacc = 1; ph[0].k = c.hidden;
      const void* qkv_mats[3] = {lw.q, lw.k, lw.v};
      const int seg_rows[3] = {q_size, kv_size, kv_size};
      const void* biases[3] = {lw.q_bias, lw.k_bias, lw.v_bias};
      int col = 0;
      for (int s = 0; s < 3; ++s) {
        ph[0].tmap[s] = tmaps_dev + 7 * l + s;
        ph[0].w[s] = static_cast<const bf16*>(qkv_mats[s]);
        ph[0].bias[s] = c.qkv_bias ? static_cast<const bf16*>(biases[s]) : nullptr;
        ph[0].n[s] = seg_rows[s];
        ph[0].out_col[s] = col;
        col += seg_rows[s];
      }
      ph[0].epi = EPI_STORE; ph[0].bmode = B_NORM; ph[0].gather = (l == 0);
      ph[0].normw = static_cast<const bf16*>(lw.input_norm);
      ph[0].src = hidden_a; ph[0].src_ld = c.hidden; ph[0].dst = qkv; ph[0].dst_ld = qkv_width(c);
      if (split) {
        ph[0].add_parts = prev_parts; ph[0].partial = partial; ph[0].h_out = hidden_b;
      }
      // o_proj; its activation operand is the attention output (bf16 or chunk partials)
      ph[1].nseg = 1; ph[1].nacc = 1; ph[1].k = q_size;
      ph[1].tmap[0] = tmaps_dev + 7 * l + 3; ph[1].w[0] = static_cast<const bf16*>(lw.o);
      ph[1].n[0] = c.hidden;
      ph[1].epi = split ? EPI_PARTIAL : EPI_RESIDUAL; ph[1].bmode = B_ATTN;
      ph[1].src = attn; ph[1].src_ld = q_size; ph[1].dst = hidden_a; ph[1].dst_ld = c.hidden;
      ph[1].partial = partial;
      // gate, up -> silu(gate) * up
      ph[2].nseg = 1; ph[2].nacc = 2; ph[2].k = c.hidden;
      ph[2].tmap[0] = tmaps_dev + 7 * l + 4; ph[2].tmap[1] = tmaps_dev + 7 * l + 5;
      ph[2].w[0] = static_cast<const bf16*>(lw.gate); ph[2].w[1] = static_cast<const bf16*>(lw.up);
      ph[2].n[0] = c.intermediate; ph[2].n[1] = c.intermediate;
      ph[2].epi = EPI_SILU; ph[2].bmode = B_NORM; ph[2].normw = static_cast<const bf16*>(lw.post_norm);
      ph[2].src = split ? hidden_b : hidden_a; ph[2].src_ld = c.hidden; ph[2].dst = act; ph[2].dst_ld = c.intermediate;
      // down
      ph[3].nseg = 1; ph[3].nacc = 1; ph[3].k = c.intermediate;
      ph[3].tmap[0] = tmaps_dev + 7 * l + 6; ph[3].w[0] = static_cast<const bf16*>(lw.down);
      ph[3].n[0] = c.hidden;
      ph[3].epi = split ? EPI_PARTIAL : EPI_RESIDUAL; ph[3].bmode = B_PLAIN;
      ph[3].src = act; ph[3].src_ld = c.intermediate; ph[3].dst = hidden_a; ph[3].dst_ld = c.hidden;
      ph[3].partial = partial;
      if (c.tp_size > 1) {  // tensor parallel: the residual add moves behind the all-reduce (tp_allreduce)
        ph[1].epi = EPI_TP; ph[1].tp_buf = 0;
        ph[3].epi = EPI_TP; ph[3].tp_buf = 1;
      }
      ph[1].gate = 1;  // decode attention streams cache tiles through the weight ring just before this phase
      for (int i = 0; i < 4; ++i) finish_phase_tc(ph[i], h->grid, split && ph[i].epi == EPI_PARTIAL, c.max_tokens);
      if (split) {
        ph[2].add_parts = ph[1].ksplit; ph[2].partial = partial; ph[2].h_out = hidden_a;
        prev_parts = ph[3].ksplit;
      }
      for (int t = 0; t < kOperandTiles; ++t) {  // token operands: normalised rows, attention output, SiLU*up
        ph[0].bmap[t] = operand_maps + OPERAND_XNORM * kOperandTiles + t;
        ph[1].bmap[t] = operand_maps + OPERAND_ATTN * kOperandTiles + t;
        ph[2].bmap[t] = operand_maps + OPERAND_XNORM * kOperandTiles + t;
        ph[3].bmap[t] = operand_maps + OPERAND_ACT * kOperandTiles + t;
      }
      // One TMA descriptor per matrix, boxed to the tile height and the K chunks per copy its phase chose.
      const void* mats[7] = {lw.q, lw.k, lw.v, lw.o, lw.gate, lw.up, lw.down};
      const int rows[7] = {q_size, kv_size, kv_size, c.hidden, c.intermediate, c.intermediate, c.hidden};
      const int ks[7] = {c.hidden, c.hidden, c.hidden, q_size, c.hidden, c.hidden, c.intermediate};
      const int which[7] = {0, 0, 0, 1, 2, 2, 3};
      for (int i = 0; i < 7; ++i)
        if (int e = encode_phase_weight_map(&tmaps_host[7 * l + i], mats[i], rows[i], ks[i], ph[which[i]], use3d)) return e;
    }
    GemmPhase& head = tp[4 * L];
    memset(&head, 0, sizeof(head));
    head.nseg = 1; head.nacc = 1; head.k = c.hidden;
    head.tmap[0] = tmaps_dev + 7 * L; head.w[0] = static_cast<const bf16*>(w->lm_head);
    head.n[0] = c.vocab;
    head.epi = EPI_STORE; head.bmode = B_NORM; head.normw = static_cast<const bf16*>(w->final_norm);
    head.src = hidden_a; head.src_ld = c.hidden; head.to_logits = 1; head.dst_ld = c.vocab;
    if (split) {
      head.add_parts = prev_parts; head.partial = partial;
    }
    finish_phase_tc(head, h->grid, false, c.max_tokens);
    for (int t = 0; t < kOperandTiles; ++t) head.bmap[t] = operand_maps + OPERAND_XNORM * kOperandTiles + t;
    if (int e = encode_phase_weight_map(&tmaps_host[7 * L], w->lm_head, c.vocab, c.hidden, head, use3d)) return e;
  }
  // Table 2: the split-K table again for the small-launch kernel, whose mma.sync consumer takes tiles of
  // at most 64 rows (four 16-row fragments) of any height below that.
  h->fma_ok = small_shape_ok(c) && h->use3d;
  for (size_t i = 0; i < nphases && h->fma_ok; ++i)
    if (phases[i].kslice > kBSlots || phases[i].rows > kTileRows) h->fma_ok = false;
  if (h->fma_ok) {
    for (size_t i = 0; i < nphases; ++i) {
      GemmPhase& ph = phases[2 * nphases + i];
      ph = phases[i];
      finish_phase(ph, h->grid, ph.epi == EPI_PARTIAL);  // any tile height: no rounding to 8
      if (ph.rows > kSmallTileRows) {
        if (ph.ksplit != 1) return fail(MK_ERR_UNSUPPORTED, "small-launch table: a split phase with more than 64 rows");
        finish_phase(ph, h->grid, false, kSmallTileRows);
      }
      if (ph.nseg == 3 || ph.nacc == 2) {  // q/k/v and gate/up: outputs leave in pairs of rows: even tile height
        if (ph.rows & 1) {
          ph.rows += 1;
          const int nsg = ph.nacc == 2 ? 1 : ph.nseg;
          int tile = 0;
          for (int sg = 0; sg < nsg; ++sg) {
            ph.tile_start[sg] = tile;
            tile += (ph.n[sg] + ph.rows - 1) / ph.rows;
          }
          ph.tile_start[nsg] = tile;
          ph.ntiles = tile;
          ph.nunits = tile * ph.ksplit;
        }
        const bool even = ph.n[0] % 2 == 0 && (ph.nacc == 2 || (ph.n[1] % 2 == 0 && ph.n[2] % 2 == 0));
        ph.ll = (ph.rows <= kSmallTileRows && even && ph.ksplit == 1) ? 1 : 0;
      }
      // One copy = one three-dimensional box: the tile's rows x kb K chunks, each chunk 128-byte swizzled
      // for ldmatrix; as many chunks as fit the copy size (a copy of less than ~16 KB cannot keep an
      // SM's share of HBM busy: the copy engine retires about three per microsecond).
      int kb = 1;
      for (int cand = 2; cand <= std::min(ph.kslice, 256); ++cand)
        if (ph.kslice % cand == 0 && ph.rows * cand * 128 <= kBoxCopyBytes) kb = cand;
      ph.kb = kb;
      ph.map3d = 1;
      ph.gran = (ph.rows * kb * 128 + kGranule - 1) / kGranule;
      const int nseg = ph.nacc == 2 ? 2 : ph.nseg;
      for (int sg = 0; sg < nseg; ++sg) {
        const size_t index = static_cast<size_t>(ph.tmap[sg] - dmaps);  // same matrix, same slot in the third set
        ph.tmap[sg] = dmaps + 2 * nmaps + index;
        if (encode_weight_map3(&maps[2 * nmaps + index], ph.w[sg], ph.n[sg], ph.k, ph.rows, kb) != MK_OK) h->fma_ok = false;
      }
    }
  }
  // Stamped hand-offs of the small-launch table (q/k/v -> attention -> o_proj, gate/up -> down): all or none.
  h->small_ll = h->fma_ok;
  for (int l = 0; l < L && h->small_ll; ++l)
    if (!phases[2 * nphases + 4 * l].ll || !phases[2 * nphases + 4 * l + 2].ll) h->small_ll = false;
  for (int l = 0; l < L && h->fma_ok; ++l) {
    GemmPhase* ph = phases.data() + 2 * nphases + 4 * l;
    for (int i = 0; i < 4; ++i) {
      ph[i].ll = 0; ph[i].ll_dst = nullptr; ph[i].ll_src = nullptr; ph[i].ll_ld = 0; ph[i].ll_src_ld = 0;
    }
    if (!h->small_ll) continue;
    ph[0].ll = 1; ph[0].ll_dst = at<unsigned long long>(h, h->cv.qkv_ll); ph[0].ll_ld = qkv_width(c) / 2;
    // o_proj reads the attention output that the first chunk's CTA of every head combined and stamped as bf16 pairs
    ph[1].ll_src = at<unsigned long long>(h, h->cv.attn_ll); ph[1].ll_src_ld = q_size / 2; ph[1].bmode = B_PLAIN;
    ph[2].ll = 1; ph[2].ll_dst = at<unsigned long long>(h, h->cv.act_ll); ph[2].ll_ld = c.intermediate / 2;
    ph[3].ll_src = at<unsigned long long>(h, h->cv.act_ll); ph[3].ll_src_ld = c.intermediate / 2;
    // with no barrier between attention and o_proj, nor gate/up and down, their partials need buffers of their own
    ph[3].partial = at<float>(h, h->cv.partial2);
    if (l + 1 < L) ph[4].partial = at<float>(h, h->cv.partial2);
  }
  if (h->fma_ok && h->small_ll) phases[2 * nphases + 4 * L].partial = at<float>(h, h->cv.partial2);  // lm_head adds the last down-proj
  // Table 3, one-token launches: o_proj and down_proj are not cut along K.  A CTA takes whole weight rows
  // (contiguous in memory, fetched by one-dimensional bulk copies of up to 28 KB), adds the residual in its
  // epilogue and stamps the new residual stream, which the next normalising phase polls: no fp32 partials,
  // no grid barrier inside a layer.  The residual stream alternates between res_a (after the MLP) and res_b.
  h->row_ok = h->small_ll && c.hidden % 2 == 0 && q_size * 2 <= h->fat_copy - 2048 && c.intermediate * 2 <= h->fat_copy - 2048 &&
              c.intermediate <= kSplitTokens * kBSlots * kChunkK && q_size <= kSplitTokens * kBSlots * kChunkK;
  if (h->row_ok) {
    unsigned long long* res_a = at<unsigned long long>(h, h->cv.res_a);
    unsigned long long* res_b = at<unsigned long long>(h, h->cv.res_b);
    // The row table's consumer runs on CUDA cores over plain rows: its box phases (q/k/v, gate/up, lm_head)
    // get descriptors of their own, boxes of kb * 64 elements x the tile's rows without swizzle.
    for (size_t i = 0; i < nphases && h->row_ok; ++i) {
      GemmPhase& ph = phases[3 * nphases + i];
      ph = phases[2 * nphases + i];
      ph.map3d = 0;
      int kb = 1;
      for (int cand = 2; cand <= 4; cand += 2)
        if (ph.kslice % cand == 0 && ph.rows * cand * 128 <= kBoxCopyBytes) kb = cand;
      ph.kb = kb;
      ph.gran = (ph.rows * kb * 128 + kGranule - 1) / kGranule;
      const int nseg = ph.nacc == 2 ? 2 : ph.nseg;
      for (int sg = 0; sg < nseg; ++sg) {
        const size_t index = static_cast<size_t>(ph.tmap[sg] - (dmaps + 2 * nmaps));
        ph.tmap[sg] = row_dmaps + index;
        if (encode_weight_map(&row_maps[index], ph.w[sg], ph.n[sg], ph.k, ph.rows, kb, false) != MK_OK) h->row_ok = false;
      }
    }
    for (int l = 0; l <= L; ++l) {
      GemmPhase* ph = phases.data() + 3 * nphases + 4 * l;
      // normalising phases read the stamped residual stream (layer 0 still gathers embedding rows)
      ph[0].add_parts = 0; ph[0].h_out = nullptr; ph[0].partial = nullptr;
      ph[0].ll_src = ph[0].gather ? nullptr : res_a; ph[0].ll_src_ld = c.hidden / 2;
      if (l == L) break;  // the lm_head phase
      ph[2].add_parts = 0; ph[2].h_out = nullptr; ph[2].partial = nullptr;
      ph[2].ll_src = res_b; ph[2].ll_src_ld = c.hidden / 2;
      for (int which = 1; which <= 3; which += 2) {
        GemmPhase& rp = ph[which];
        rp.ksplit = 1; rp.kslice = rp.kc;
        rp.rows = choose_rows(rp, h->grid, kSmallTileRows);
        if (rp.rows & 1) rp.rows += 1;
        rp.tile_start[0] = 0;
        rp.ntiles = (rp.n[0] + rp.rows - 1) / rp.rows;
        rp.tile_start[1] = rp.ntiles;
        rp.nunits = rp.ntiles;
        rp.bulk = 1;
        const int row_bytes = rp.k * 2;
        rp.rpc = std::max(1, std::min(8, (h->fat_copy - 2048) / row_bytes));
        if (rp.rpc > rp.rows) rp.rpc = rp.rows;
        rp.kb = 1;
        rp.gran = (rp.rpc * row_bytes + kGranule - 1) / kGranule;
        rp.epi = EPI_ROWRES; rp.partial = nullptr;
        rp.ll = 1; rp.ll_ld = c.hidden / 2;
        rp.res_src = (which == 1) ? res_a : res_b;   // layer 0's o_proj adds the embedding row (rp.gather below)
        rp.ll_dst = (which == 1) ? res_b : res_a;
        rp.gather = (which == 1 && l == 0) ? 1 : 0;
      }
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    CUtensorMap operand_host[kOperandMaps];
    memset(operand_host, 0, sizeof(operand_host));
    const void* bases[3] = {at<bf16>(h, h->cv.xnorm), attn, act};
    const int widths[3] = {c.hidden, q_size, c.intermediate};
    static const int tiles[kOperandTiles] = {16, 32, 64, 128};
    for (int kind = 0; kind < 3; ++kind)
      for (int t = 0; t < kOperandTiles; ++t)
        if (int e = encode_operand_map(&operand_host[kind * kOperandTiles + t], bases[kind], c.max_tokens, widths[kind], tiles[t])) return e;
    MK_CUDA(cudaMemcpyAsync(operand_maps, operand_host, sizeof(operand_host), cudaMemcpyHostToDevice, s));
    MK_CUDA(cudaStreamSynchronize(s));
  }
  MK_CUDA(cudaMemcpyAsync(dmaps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, s));
  MK_CUDA(cudaMemcpyAsync(row_dmaps, row_maps.data(), row_maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, s));
  MK_CUDA(cudaMemcpyAsync(at<GemmPhase>(h, h->cv.phases), phases.data(), phases.size() * sizeof(GemmPhase),
                          cudaMemcpyHostToDevice, s));
  // The source vectors die at return: make sure the copies have read them.
  MK_CUDA(cudaStreamSynchronize(s));
  h->layers.assign(w->layers, w->layers + L);
  h->weights = *w;
  h->weights.layers = h->layers.data();
  h->bound = true;
  return MK_OK;
}

namespace {
// Keys the small-launch kernel's 16 KB score buffer covers: at most 16 context chunks of 4096 / group keys.
int small_launch_keys(const mk_config& c) { return kMaxChunks * ((kAttScoreBytes / 4 / (c.q_heads / c.kv_heads)) & ~7); }

bool small_launch_ok(mk_handle h, int capacity) {
  return (h->cfg.engine == MK_ENGINE_FMA || h->cfg.engine == MK_ENGINE_AUTO) && small_shape_ok(h->cfg) && h->fma_ok &&
         capacity <= small_launch_keys(h->cfg);
}

int decode_once(mk_handle h, const int64_t* ids, const int64_t* positions, int batch, void* const* key_caches,
                void* const* value_caches, int32_t* const* valid_lengths, int capacity, void* logits, void* stream,
                int64_t* tokens_out = nullptr, bool sample = false, bool ragged = false);

}  // namespace

namespace {
// One decode step (mk_decode), or one step of mk_decode_steps (`sample`: the kernel picks the greedy
// tokens, stores them in tokens_out and as the next ids, and advances the positions).  Lock held.
int decode_step(mk_handle h, const int64_t* ids, const int64_t* positions, int batch, void* const* key_caches,
                void* const* value_caches, int32_t* const* valid_lengths, int capacity, void* logits, void* stream,
                int64_t* tokens_out, bool sample);
}  // namespace

int mk_decode(mk_handle h, const int64_t* ids, const int64_t* positions, int batch, void* const* key_caches,
              void* const* value_caches, int32_t* const* valid_lengths, int capacity, void* logits, void* stream) {
  if (!h || !ids || !positions || !key_caches || !value_caches || !valid_lengths || !logits)
    return fail(MK_ERR_INVALID, "mk_decode: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  return decode_step(h, ids, positions, batch, key_caches, value_caches, valid_lengths, capacity, logits, stream, nullptr, false);
}

int mk_decode_ragged(mk_handle h, const int64_t* ids, const int64_t* positions, int batch, void* const* key_caches,
                     void* const* value_caches, int32_t* const* valid_lengths, int capacity, void* logits, void* stream) {
  if (!h || !ids || !positions || !key_caches || !value_caches || !valid_lengths || !logits)
    return fail(MK_ERR_INVALID, "mk_decode_ragged: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  if (!h->bound) return fail(MK_ERR_UNBOUND, "mk_decode_ragged before mk_bind_weights");
  if (batch < 1 || batch > h->cfg.max_tokens) return fail(MK_ERR_INVALID, "mk_decode_ragged: batch %d outside [1, %d]", batch, h->cfg.max_tokens);
  if (capacity < 1) return fail(MK_ERR_INVALID, "mk_decode_ragged: capacity %d", capacity);
  if (int e = attention_fits(h, capacity, "mk_decode_ragged")) return e;
  for (int l = 0; l < h->cfg.layers; ++l) {
    if (!key_caches[l] || !value_caches[l] || !valid_lengths[l]) return fail(MK_ERR_INVALID, "mk_decode_ragged: layer %d state is null", l);
    if (reinterpret_cast<uintptr_t>(key_caches[l]) % 16 || reinterpret_cast<uintptr_t>(value_caches[l]) % 16)
      return fail(MK_ERR_ALIGNMENT, "mk_decode_ragged: layer %d cache is not 16-byte aligned", l);
  }
  return decode_once(h, ids, positions, batch, key_caches, value_caches, valid_lengths, capacity, logits, stream, nullptr, false, true);
}

int mk_decode_steps(mk_handle h, int64_t* ids, int64_t* positions, int batch, void* const* key_caches,
                    void* const* value_caches, int32_t* const* valid_lengths, int capacity, int steps, int64_t* tokens_out,
                    void* logits, void* stream) {
  if (!h || !ids || !positions || !key_caches || !value_caches || !valid_lengths || !logits || !tokens_out)
    return fail(MK_ERR_INVALID, "mk_decode_steps: null argument");
  if (steps < 1) return fail(MK_ERR_INVALID, "mk_decode_steps: steps %d", steps);
  std::lock_guard<std::mutex> guard(h->lock);
  for (int step = 0; step < steps; ++step)
    if (int e = decode_step(h, ids, positions, batch, key_caches, value_caches, valid_lengths, capacity, logits, stream,
                            tokens_out + static_cast<size_t>(step) * batch, true))
      return e;
  return MK_OK;
}

int mk_decode_step_host(mk_handle h, const int64_t* host_ids, const int64_t* host_positions, int batch,
                        void* const* key_caches, void* const* value_caches, int32_t* const* valid_lengths, int capacity,
                        void* logits, int64_t* host_tokens_out, void* stream) {
  if (!h || !host_ids || !host_positions || !key_caches || !value_caches || !valid_lengths || !logits || !host_tokens_out)
    return fail(MK_ERR_INVALID, "mk_decode_step_host: null argument");
  if (batch < 1 || batch > h->cfg.max_tokens)
    return fail(MK_ERR_INVALID, "mk_decode_step_host: batch %d outside [1, %d]", batch, h->cfg.max_tokens);
  std::lock_guard<std::mutex> guard(h->lock);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t* io = at<int64_t>(h, h->cv.host_io);
  int64_t *ids = io, *positions = io + h->cfg.max_tokens, *tokens = io + 2 * static_cast<size_t>(h->cfg.max_tokens);
  const size_t bytes = static_cast<size_t>(batch) * sizeof(int64_t);
  MK_CUDA(cudaMemcpyAsync(ids, host_ids, bytes, cudaMemcpyHostToDevice, s));
  MK_CUDA(cudaMemcpyAsync(positions, host_positions, bytes, cudaMemcpyHostToDevice, s));
  if (int e = decode_step(h, ids, positions, batch, key_caches, value_caches, valid_lengths, capacity, logits, stream, tokens, true))
    return e;
  MK_CUDA(cudaMemcpyAsync(host_tokens_out, tokens, bytes, cudaMemcpyDeviceToHost, s));
  MK_CUDA(cudaStreamSynchronize(s));
  return MK_OK;
}

namespace {
int decode_step(mk_handle h, const int64_t* ids, const int64_t* positions, int batch, void* const* key_caches,
                void* const* value_caches, int32_t* const* valid_lengths, int capacity, void* logits, void* stream,
                int64_t* tokens_out, bool sample) {
  if (!h->bound) return fail(MK_ERR_UNBOUND, "mk_decode before mk_bind_weights");
  if (batch < 1 || batch > h->cfg.max_tokens) return fail(MK_ERR_INVALID, "mk_decode: batch %d outside [1, %d]", batch, h->cfg.max_tokens);
  if (capacity < 1) return fail(MK_ERR_INVALID, "mk_decode: capacity %d", capacity);
  if (int e = attention_fits(h, capacity, "mk_decode")) return e;
  const int L = h->cfg.layers;
  for (int l = 0; l < L; ++l) {
    if (!key_caches[l] || !value_caches[l] || !valid_lengths[l]) return fail(MK_ERR_INVALID, "mk_decode: layer %d state is null", l);
    if (reinterpret_cast<uintptr_t>(key_caches[l]) % 16 || reinterpret_cast<uintptr_t>(value_caches[l]) % 16)
      return fail(MK_ERR_ALIGNMENT, "mk_decode: layer %d cache is not 16-byte aligned", l);
  }
  return decode_once(h, ids, positions, batch, key_caches, value_caches, valid_lengths, capacity, logits, stream, tokens_out, sample);
}
}  // namespace

namespace {
int decode_once(mk_handle h, const int64_t* ids, const int64_t* positions, int batch, void* const* key_caches,
                void* const* value_caches, int32_t* const* valid_lengths, int capacity, void* logits, void* stream,
                int64_t* tokens_out, bool sample, bool ragged) {
  KParams p;
  base_params(h, p);
  const int L = h->cfg.layers;
  for (int l = 0; l < L; ++l) {
    p.kc[l] = key_caches[l];
    p.vc[l] = value_caches[l];
    p.len[l] = valid_lengths[l];
  }
  const int ntt = token_tiles(batch);
  p.mode = MODE_DECODE; p.m = batch; p.batch = batch; p.seq = 1; p.capacity = capacity;
  p.split = split_table_ok(h->cfg) ? 1 : 0;
  p.phases = at<GemmPhase>(h, h->cv.phases) + (p.split ? 0 : phases_per_table(h->cfg));
  const bool small = !ragged && batch <= kSplitTokens && small_launch_ok(h, capacity);
  p.ragged = ragged ? 1 : 0;
  if (!small && h->kv_maps_ok) {
    // Tiled descriptors of the caches for the tensor engine's decode attention, encoded again only when a
    // cache pointer or the geometry differs from the last call's (the copy is ordered on `stream`
    // before the launch; its pageable source is staged before cudaMemcpyAsync returns).
    const mk_config& c = h->cfg;
    const int gs = c.q_heads / c.kv_heads, row_elems = c.kv_heads * c.head_dim;
    const int hpu = decode_heads_per_unit(c.kv_heads, gs, c.head_dim);
    const int tile_keys = kDecTileBytes / (c.head_dim * 2 * hpu);
    const bool shape_ok = (hpu & (hpu - 1)) == 0 && tile_keys % 16 == 0 && tile_keys <= 256 && c.head_dim % kChunkK == 0;
    int slot = -1, oldest = 0;
    for (int i = 0; i < kCacheMapSets && shape_ok && slot < 0; ++i) {
      const auto& set = h->kv_sets[i];
      if (set.used < h->kv_sets[oldest].used) oldest = i;
      bool same = static_cast<int>(set.seen.size()) == 2 * L && set.capacity == capacity && set.batch == batch;
      for (int l = 0; l < L && same; ++l) same = set.seen[l] == key_caches[l] && set.seen[L + l] == value_caches[l];
      if (same) slot = i;
    }
    CUtensorMap* const device_sets = at<CUtensorMap>(h, h->cv.kvmaps);
    if (shape_ok && slot < 0) {
      std::vector<CUtensorMap> fresh(2 * static_cast<size_t>(L));
      bool encoded = true;
      for (int l = 0; l < L && encoded; ++l) {
        encoded = encode_cache_map(&fresh[l], key_caches[l], batch, capacity, row_elems, tile_keys, hpu * (c.head_dim / kChunkK)) == MK_OK &&
                  encode_cache_map(&fresh[L + l], value_caches[l], batch, capacity, row_elems, tile_keys, hpu * (c.head_dim / kChunkK)) == MK_OK;
      }
      if (encoded) {
        slot = oldest;
        MK_CUDA(cudaMemcpyAsync(device_sets + static_cast<size_t>(slot) * 2 * L, fresh.data(), fresh.size() * sizeof(CUtensorMap),
                                cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
        auto& set = h->kv_sets[slot];
        set.seen.assign(2 * static_cast<size_t>(L), nullptr);
        for (int l = 0; l < L; ++l) {
          set.seen[l] = key_caches[l];
          set.seen[L + l] = value_caches[l];
        }
        set.capacity = capacity;
        set.batch = batch;
      } else {
        h->kv_maps_ok = false;  // this driver refuses the view: plain copies from here on
      }
    }
    if (slot >= 0) {
      h->kv_sets[slot].used = static_cast<uint64_t>(h->launches) + 1;
      p.kv_maps = device_sets + static_cast<size_t>(slot) * 2 * L;
    }
  }
  if (small) p.phases = at<GemmPhase>(h, h->cv.phases) + 2 * phases_per_table(h->cfg);
  p.n_gemm = 4 * L + 1;
  p.nbar = 7 * L + 1;  // tensor engine: five per layer and one behind each norm phase (two per layer, one for the lm_head)
  if (small) p.nbar = 5 * L;
  if (small && h->small_ll) p.nbar = 2 * L;  // stamped hand-offs: only o_proj -> gate/up and down -> next layer keep a grid barrier
  if (small && h->row_ok && batch == 1) {     // one token: the row table, a single grid barrier at the very end
    p.phases = at<GemmPhase>(h, h->cv.phases) + 3 * phases_per_table(h->cfg);
    p.nbar = 1;
    p.rowmode = 1;
  }
  p.small_ring = small_ring_for(h, p.rowmode ? 1 : 2);
  p.stream_once = (ntt == 1);
  p.ids = reinterpret_cast<long long*>(const_cast<int64_t*>(ids));
  p.pos = reinterpret_cast<long long*>(const_cast<int64_t*>(positions));
  p.logits = static_cast<bf16*>(logits);
  if (p.tp_size > 1) {
    if (!h->tp_bound) return fail(MK_ERR_UNBOUND, "mk_decode: tensor-parallel handle without mk_tp_bind");
    if (sample) return fail(MK_ERR_UNSUPPORTED, "mk_decode_steps: the device-side sampler needs the whole vocabulary on one rank");
    p.nbar += 2 * L;  // one more grid barrier behind each of the two all-reduces of a layer
  }
  if (sample) {
    p.sample = 1;
    p.tokens_out = reinterpret_cast<long long*>(tokens_out);
    if (!p.rowmode) p.nbar += 1;  // the sampler runs behind one more grid barrier (the row table already ends with one)
  }
  if (int e = launch(h, p, stream, L, small)) return e;
  if (p.tp_size > 1) h->tp_epoch += 2u * static_cast<uint32_t>(L);
  return MK_OK;
}
}  // namespace

int mk_prefill(mk_handle h, const int64_t* ids, const int64_t* positions, const void* mask, int batch, int sequence,
               void* logits, void* stream) {
  if (!h || !ids || !positions || !logits) return fail(MK_ERR_INVALID, "mk_prefill: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  if (!h->bound) return fail(MK_ERR_UNBOUND, "mk_prefill before mk_bind_weights");
  const long long m = static_cast<long long>(batch) * sequence;
  if (batch < 1 || sequence < 1 || m > h->cfg.max_tokens)
    return fail(MK_ERR_INVALID, "mk_prefill: %d x %d tokens outside [1, %d]", batch, sequence, h->cfg.max_tokens);
  if (int e = attention_fits(h, sequence, "mk_prefill")) return e;
  const int gs = h->cfg.q_heads / h->cfg.kv_heads;
  if (sequence > ((kScoreBytes / 4 / gs) & ~7))
    return fail(MK_ERR_UNSUPPORTED, "mk_prefill: sequence %d exceeds the per-row score buffer", sequence);
  KParams p;
  base_params(h, p);
  const int L = h->cfg.layers;
  const int ntt = token_tiles(static_cast<int>(m));
  p.mode = MODE_PREFILL; p.m = static_cast<int>(m); p.batch = batch; p.seq = sequence; p.capacity = 0;
  p.split = split_table_ok(h->cfg) ? 1 : 0;
  p.phases = at<GemmPhase>(h, h->cv.phases) + (p.split ? 0 : phases_per_table(h->cfg));
  p.n_gemm = 4 * L + 1;
  p.nbar = 8 * L + 1;  // as decode, plus one behind the rotation of q and k
  p.stream_once = (ntt == 1);
  p.ids = reinterpret_cast<long long*>(const_cast<int64_t*>(ids));
  p.pos = reinterpret_cast<long long*>(const_cast<int64_t*>(positions));
  p.mask = static_cast<const bf16*>(mask);
  p.logits = static_cast<bf16*>(logits);
  if (p.tp_size > 1) {
    if (!h->tp_bound) return fail(MK_ERR_UNBOUND, "mk_prefill: tensor-parallel handle without mk_tp_bind");
    p.nbar += 2 * L;
  }
  if (int e = launch(h, p, stream)) return e;
  if (p.tp_size > 1) h->tp_epoch += 2u * static_cast<uint32_t>(L);
  return MK_OK;
}

int mk_linear(mk_handle h, const void* x, const void* weight, const void* bias, void* y, int m, int n, int k,
              void* stream) {
  if (!h || !x || !weight || !y) return fail(MK_ERR_INVALID, "mk_linear: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  if (m < 1 || m > h->cfg.max_tokens) return fail(MK_ERR_INVALID, "mk_linear: m %d outside [1, %d]", m, h->cfg.max_tokens);
  if (n < 1 || k < 64 || k % 64) return fail(MK_ERR_UNSUPPORTED, "mk_linear: k must be a positive multiple of 64");
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(y) % 2)
    return fail(MK_ERR_ALIGNMENT, "mk_linear: x must be 16-byte aligned");
  KParams p;
  base_params(h, p);
  GemmPhase& ph = p.linear_phase;
  memset(&ph, 0, sizeof(ph));
  ph.nseg = 1; ph.nacc = 1; ph.k = k;
  ph.w[0] = static_cast<const bf16*>(weight); ph.bias[0] = static_cast<const bf16*>(bias);
  ph.n[0] = n;
  ph.epi = EPI_STORE; ph.bmode = B_PLAIN;
  ph.src = static_cast<const bf16*>(x); ph.src_ld = k;
  ph.dst = static_cast<bf16*>(y); ph.dst_ld = n;
  finish_phase_tc(ph, h->grid, false, h->cfg.max_tokens);
  // Phase and descriptors go into the kernel's parameter block: nothing is uploaded, nothing synchronised.
  bool use3d = h->use3d;
  if (int e = encode_phase_weight_map(&p.linear_wmap, weight, n, k, ph, use3d)) return e;
  if (int e = encode_operand_map(&p.linear_xmap, x, m, k, token_tile_of(m))) return e;
  p.phases = nullptr;
  p.mode = MODE_LINEAR; p.m = m; p.batch = m; p.seq = 1;
  p.n_gemm = 1;
  p.nbar = 0;
  p.stream_once = (token_tiles(m) == 1);
  return launch(h, p, stream);
}

int mk_kv_attention(mk_handle h, const void* query, const void* key, const void* value, void* key_cache,
                    void* value_cache, int32_t* valid_length, int batch, int capacity, void* output, void* stream) {
  if (!h || !query || !key || !value || !key_cache || !value_cache || !valid_length || !output)
    return fail(MK_ERR_INVALID, "mk_kv_attention: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  if (batch < 1 || batch > h->cfg.max_tokens) return fail(MK_ERR_INVALID, "mk_kv_attention: batch %d outside [1, %d]", batch, h->cfg.max_tokens);
  if (int e = attention_fits(h, capacity, "mk_kv_attention")) return e;
  if (reinterpret_cast<uintptr_t>(key_cache) % 16 || reinterpret_cast<uintptr_t>(value_cache) % 16)
    return fail(MK_ERR_ALIGNMENT, "mk_kv_attention: caches must be 16-byte aligned");
  KParams p;
  base_params(h, p);
  p.mode = MODE_KVATT; p.m = batch; p.batch = batch; p.seq = 1; p.capacity = capacity;
  p.n_gemm = 0; p.nbar = 1;
  p.op_q = static_cast<const bf16*>(query); p.op_k = static_cast<const bf16*>(key); p.op_v = static_cast<const bf16*>(value);
  p.op_out = static_cast<bf16*>(output);
  p.kc[0] = key_cache; p.vc[0] = value_cache; p.len[0] = valid_length;
  return launch(h, p, stream, 1);
}

int mk_attention(mk_handle h, const void* query, const void* key, const void* value, const void* mask, float scale,
                 int batch, int q_len, int k_len, void* output, void* stream) {
  if (!h || !query || !key || !value || !output) return fail(MK_ERR_INVALID, "mk_attention: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  if (batch < 1 || q_len < 1 || k_len < 1) return fail(MK_ERR_INVALID, "mk_attention: sizes must be positive");
  const int gs = h->cfg.q_heads / h->cfg.kv_heads;
  if (k_len > ((kScoreBytes / 4 / gs) & ~7))
    return fail(MK_ERR_UNSUPPORTED, "mk_attention: %d keys exceed the per-row score buffer", k_len);
  if (reinterpret_cast<uintptr_t>(key) % 16 || reinterpret_cast<uintptr_t>(value) % 16)
    return fail(MK_ERR_ALIGNMENT, "mk_attention: key/value must be 16-byte aligned");
  KParams p;
  base_params(h, p);
  p.mode = MODE_ATT; p.m = batch * q_len; p.batch = batch; p.seq = q_len;
  p.n_gemm = 0; p.nbar = 0;
  p.att_scale = scale;
  p.op_q = static_cast<const bf16*>(query); p.op_k = static_cast<const bf16*>(key); p.op_v = static_cast<const bf16*>(value);
  p.op_out = static_cast<bf16*>(output);
  p.mask = static_cast<const bf16*>(mask);
  p.op_qlen = q_len; p.op_klen = k_len;
  return launch(h, p, stream);
}

int mk_status(mk_handle h, void* stream, mk_status_info* out) {
  if (!h) return fail(MK_ERR_INVALID, "mk_status: null handle");
  std::lock_guard<std::mutex> guard(h->lock);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MK_CUDA(cudaStreamSynchronize(s));
  Control c;
  MK_CUDA(cudaMemcpy(&c, at<Control>(h, h->cv.ctrl), sizeof(c), cudaMemcpyDeviceToHost));
  if (out) {
    out->status = c.status; out->where = c.where; out->cta = c.cta; out->detail = c.detail;
  }
  if (c.status != MK_STATUS_OK || c.abort) {
    // Counters are in an unknown state after an aborted launch: start over.
    MK_CUDA(cudaMemset(at<Control>(h, h->cv.ctrl), 0, sizeof(Control)));
    h->epoch = 0;
    if (h->mirror) *h->mirror = 0;
    return fail(MK_ERR_DEVICE_STATUS, "device status %d at site %d (cta %d, detail %d)", c.status, c.where, c.cta, c.detail);
  }
  return MK_OK;
}

int mk_set_status_mirror(mk_handle h, int32_t* host_word) {
  if (!h) return fail(MK_ERR_INVALID, "mk_set_status_mirror: null handle");
  std::lock_guard<std::mutex> guard(h->lock);
  if (host_word) {
    void* device_view = nullptr;
    MK_CUDA(cudaHostGetDevicePointer(&device_view, host_word, 0));  // fails unless the word is pinned, mapped host memory
    *host_word = 0;
    h->mirror = static_cast<volatile int*>(device_view);
  } else {
    h->mirror = nullptr;
  }
  return MK_OK;
}

size_t mk_tp_exchange_bytes(const mk_config* config) {
  if (!config || check_config(*config) != MK_OK || config->tp_size < 2) return 0;
  return kTpFlagBytes + 2 * static_cast<size_t>(config->tp_size) * config->max_tokens * config->hidden * sizeof(float);
}

int mk_tp_bind(mk_handle h, void* const* exchange, size_t exchange_bytes, void* stream) {
  if (!h || !exchange) return fail(MK_ERR_INVALID, "mk_tp_bind: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  const mk_config& c = h->cfg;
  if (c.tp_size < 2) return fail(MK_ERR_INVALID, "mk_tp_bind: the handle was not created for a tensor-parallel group");
  if (exchange_bytes < mk_tp_exchange_bytes(&c))
    return fail(MK_ERR_WORKSPACE, "mk_tp_bind: exchange buffers have %zu bytes, %zu needed", exchange_bytes, mk_tp_exchange_bytes(&c));
  for (int r = 0; r < c.tp_size; ++r) {
    if (!exchange[r]) return fail(MK_ERR_INVALID, "mk_tp_bind: rank %d has no exchange buffer", r);
    if (reinterpret_cast<uintptr_t>(exchange[r]) % 256) return fail(MK_ERR_ALIGNMENT, "mk_tp_bind: exchange buffers must be 256-byte aligned");
    h->tp_peer[r] = static_cast<uint8_t*>(exchange[r]);
  }
  // This rank's own flags start at zero; stamps count up from one.  (Every rank clears its own before any launch:
  // the caller synchronises the group between mk_tp_bind and the first decode.)
  MK_CUDA(cudaMemsetAsync(h->tp_peer[c.tp_rank], 0, kTpFlagBytes, static_cast<cudaStream_t>(stream)));
  h->tp_epoch = 0;
  h->tp_bound = true;
  return MK_OK;
}

int mk_ipc_export(void* pointer, mk_ipc_handle* out) {
  if (!pointer || !out) return fail(MK_ERR_INVALID, "mk_ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) <= sizeof(out->bytes), "handle does not fit");
  cudaIpcMemHandle_t handle;
  MK_CUDA(cudaIpcGetMemHandle(&handle, pointer));
  CUdeviceptr base = 0;
  size_t size = 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult found;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &found) != cudaSuccess ||
      found != cudaDriverEntryPointSuccess)
    return fail(MK_ERR_CUDA, "cuMemGetAddressRange is not available from this driver");
  const CUresult r = reinterpret_cast<CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr)>(fn)(
      &base, &size, reinterpret_cast<CUdeviceptr>(pointer));
  if (r != CUDA_SUCCESS) return fail(MK_ERR_CUDA, "cuMemGetAddressRange failed with %d", static_cast<int>(r));
  memset(out, 0, sizeof(*out));
  memcpy(out->bytes, &handle, sizeof(handle));
  out->offset = static_cast<uint64_t>(reinterpret_cast<CUdeviceptr>(pointer) - base);
  return MK_OK;
}

int mk_ipc_open(const mk_ipc_handle* in, void** pointer, void** base_out) {
  if (!in || !pointer || !base_out) return fail(MK_ERR_INVALID, "mk_ipc_open: null argument");
  cudaIpcMemHandle_t handle;
  memcpy(&handle, in->bytes, sizeof(handle));
  void* base = nullptr;
  MK_CUDA(cudaIpcOpenMemHandle(&base, handle, cudaIpcMemLazyEnablePeerAccess));
  *base_out = base;
  *pointer = static_cast<uint8_t*>(base) + in->offset;
  return MK_OK;
}

int mk_ipc_close(void* base) {
  if (!base) return MK_OK;
  MK_CUDA(cudaIpcCloseMemHandle(base));
  return MK_OK;
}

int mk_describe(mk_handle h, char* buffer, size_t bytes) {
  if (!h || !buffer || bytes == 0) return fail(MK_ERR_INVALID, "mk_describe: null argument");
  std::lock_guard<std::mutex> guard(h->lock);
  size_t used = 0;
  auto add = [&](const char* fmt, ...) {
    if (used >= bytes) return;
    va_list ap;
    va_start(ap, fmt);
    const int n = vsnprintf(buffer + used, bytes - used, fmt, ap);
    va_end(ap);
    if (n > 0) used += static_cast<size_t>(n);
  };
  add("ctas %d, weight copies %s, small-launch tables %s/%s/%s, tp %d/%d\n", h->grid,
      h->use3d ? "3-D (several K chunks per copy)" : "2-D (one K chunk per copy)", h->fma_ok ? "split-K" : "-",
      h->small_ll ? "stamped" : "-", h->row_ok ? "rows" : "-", h->cfg.tp_size > 1 ? h->cfg.tp_rank : 0,
      h->cfg.tp_size > 1 ? h->cfg.tp_size : 1);
  if (h->bound) {
    std::vector<GemmPhase> phases(phases_per_table(h->cfg) * 4);
    MK_CUDA(cudaMemcpy(phases.data(), at<GemmPhase>(h, h->cv.phases), phases.size() * sizeof(GemmPhase), cudaMemcpyDeviceToHost));
    static const char* names[5] = {"qkv", "o", "gate/up", "down", "lm_head"};
    for (int table = 0; table < 4; ++table) {
      if (table == 0 && !split_table_ok(h->cfg)) continue;
      if (table == 2 && !h->fma_ok) continue;
      if (table == 3 && !h->row_ok) continue;
      add("table %d:", table);
      for (int i = 0; i < 5; ++i) {
        const GemmPhase& ph = phases[table * phases_per_table(h->cfg) + (i < 4 ? i : 4 * h->cfg.layers)];
        add(" %s rows %d ksplit %d kb %d units %d;", names[i], ph.rows, ph.ksplit, ph.kb, ph.nunits);
      }
      add("\n");
    }
  }
  return MK_OK;
}

int mk_debug_skew_barrier(mk_handle h, uint32_t delta) {
  if (!h) return fail(MK_ERR_INVALID, "mk_debug_skew_barrier: null handle");
  std::lock_guard<std::mutex> guard(h->lock);
  h->epoch += delta;
  return MK_OK;
}

int mk_set_trace(mk_handle h, void* buffer, int events_per_cta) {
  if (!h) return fail(MK_ERR_INVALID, "mk_set_trace: null handle");
  if (buffer && events_per_cta < 1) return fail(MK_ERR_INVALID, "mk_set_trace: events_per_cta must be positive");
  std::lock_guard<std::mutex> guard(h->lock);
  h->trace = static_cast<unsigned long long*>(buffer);
  h->trace_cap = buffer ? events_per_cta : 0;
  return MK_OK;
}

int mk_launch_info(mk_handle h, int32_t* ctas, int32_t* smem_bytes, int64_t* launches) {
  if (!h) return fail(MK_ERR_INVALID, "mk_launch_info: null handle");
  if (ctas) *ctas = h->grid;
  if (smem_bytes) *smem_bytes = kSmemBytes;
  if (launches) *launches = h->launches;
  return MK_OK;
}


}  // extern "C"

// ---------------------------------------------------------------------------
// mk_kv_attention_static: the stand-alone decode attention on scratch that lives
// in the library image instead of in a caller workspace.
//
// Who needs it: a caller that may not obtain device memory at the point of the
// call -- a serving process that handed all of its HBM to its own pool at start
// and forbids later allocations so a request can never fail or stall on one, or
// a call site inside a latency-critical loop where an allocation would
// serialise the device.  Such a caller has no workspace to give mk_create, so
// the exchange buffers of the split-context attention live in a fixed array of
// the module, sized for small decode batches.
constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

constexpr int kStaticDevices = 16;

struct StaticSlot {
  bool ready = false;
  uint8_t* base = nullptr;   // device address of g_static_scratch on this device
  int grid = 0;
  long long timeout_cycles = 0;
  uint32_t epoch = 0, att_epoch = 0;
  int64_t launches = 0;
  std::mutex lock;
};
StaticSlot g_static_slots[kStaticDevices];

// Scratch layout: control block, (max, sum, stamp) exchange, fp32 chunk partials.
struct StaticLayout { size_t ctrl, att_xch, att_part, total; };

StaticLayout static_layout(int batch, int q_heads, int kv_heads, int head_dim) {
  StaticLayout v{};
  v.ctrl = 0;
  v.att_xch = align_up(sizeof(Control), 256);
  v.att_part = align_up(v.att_xch + static_cast<size_t>(batch) * kv_heads * kMaxChunks * kExchangeFloats * 4, 256);
  v.total = align_up(v.att_part + static_cast<size_t>(batch) * q_heads * kMaxChunks * head_dim * 4, 256);
  return v;
}

// One-time set-up per device: symbol address, launch attributes, zeroed scratch.
int static_setup(StaticSlot& slot, int device, cudaStream_t stream) {
  int major = 0, coop = 0, khz = 0, sms = 0;
  MK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  MK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
  MK_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device));
  MK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  if (major != 10) return fail(MK_ERR_UNSUPPORTED, "device %d is sm_%d0; this library is built for sm_100a only", device, major);
  if (!coop) return fail(MK_ERR_UNSUPPORTED, "device %d does not support cooperative launch", device);
  void* address = nullptr;
  const cudaError_t found = cudaGetSymbolAddress(&address, g_static_scratch);
  if (found != cudaSuccess || !address)
    return fail(MK_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", device, cudaGetErrorString(found));
  MK_CUDA(cudaFuncSetAttribute(megakernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  MK_CUDA(cudaFuncSetAttribute(megakernel, cudaFuncAttributePreferredSharedMemoryCarveout, (kSmemBytes * 100 + 233471) / 233472));
  int per_sm = 0;
  MK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, megakernel, kThreads, kSmemBytes));
  if (per_sm < 1) return fail(MK_ERR_UNSUPPORTED, "the megakernel does not fit on an SM of device %d", device);
  // Barrier counter, abort flag, status word and every exchange stamp must start at zero.
  MK_CUDA(cudaMemsetAsync(address, 0, kStaticScratchBytes, stream));
  double ms = 2000.0;
  if (const char* env = getenv("MEGABAKE_WAIT_LIMIT_MS")) ms = atof(env) > 0 ? atof(env) : ms;
  slot.base = static_cast<uint8_t*>(address);
  slot.grid = sms;
  slot.timeout_cycles = static_cast<long long>(ms * static_cast<double>(khz));
  slot.epoch = slot.att_epoch = 0;
  slot.launches = 0;
  slot.ready = true;
  return MK_OK;
}

}  // namespace

extern "C" {

// The status word and the abort flag of the static array, which no handle owns: synchronises
// `stream`, copies them out and, if a launch was refused or gave up a wait, clears them and
// restarts the barrier count, so that the next mk_kv_attention_static call on the device works
// again (without this a timed-out wait would leave the abort flag set for the life of the process
// and every later call would return at its first wait).  Allocates nothing.
int mk_kv_attention_static_status(int device, void* stream, mk_status_info* out) {
  if (device < 0 || device >= kStaticDevices)
    return fail(MK_ERR_INVALID, "mk_kv_attention_static_status: device %d outside [0, %d)", device, kStaticDevices);
  int current = -1;
  MK_CUDA(cudaGetDevice(&current));
  if (current != device)
    return fail(MK_ERR_INVALID, "mk_kv_attention_static_status: device %d is not the current device (%d)", device, current);
  StaticSlot& slot = g_static_slots[device];
  std::lock_guard<std::mutex> guard(slot.lock);
  if (out) out->status = out->where = out->cta = out->detail = 0;
  if (!slot.ready) return MK_OK;  // nothing has run on this device yet
  MK_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  Control c;
  MK_CUDA(cudaMemcpy(&c, slot.base, sizeof(c), cudaMemcpyDeviceToHost));
  if (out) {
    out->status = c.status; out->where = c.where; out->cta = c.cta; out->detail = c.detail;
  }
  if (c.status != MK_STATUS_OK || c.abort) {
    MK_CUDA(cudaMemset(slot.base, 0, sizeof(Control)));
    slot.epoch = 0;
    return fail(MK_ERR_DEVICE_STATUS, "static scratch: device status %d at site %d (cta %d, detail %d)", c.status, c.where,
                c.cta, c.detail);
  }
  return MK_OK;
}

// Overlapping calls on one device (two streams, two threads) share the scratch and race:
// callers serialise them.  The first call on a device does the set-up (symbol lookup,
// function attributes, clearing the scratch on `stream`); make it before any stream capture.
int mk_kv_attention_static(int q_heads, int kv_heads, int head_dim, const void* query, const void* key,
                           const void* value, void* key_cache, void* value_cache, int32_t* valid_length, int batch,
                           int capacity, void* output, int device, void* stream) {
  if (!query || !key || !value || !key_cache || !value_cache || !valid_length || !output)
    return fail(MK_ERR_INVALID, "mk_kv_attention_static: null argument");
  if (device < 0 || device >= kStaticDevices)
    return fail(MK_ERR_INVALID, "mk_kv_attention_static: device %d outside [0, %d)", device, kStaticDevices);
  if (batch < 1 || capacity < 1 || q_heads < 1 || kv_heads < 1)
    return fail(MK_ERR_INVALID, "mk_kv_attention_static: sizes must be positive");
  if (head_dim != 64 && head_dim != 128) return fail(MK_ERR_UNSUPPORTED, "mk_kv_attention_static: head_dim must be 64 or 128");
  if (q_heads % kv_heads || q_heads / kv_heads > 8)
    return fail(MK_ERR_UNSUPPORTED, "mk_kv_attention_static: q_heads must be 1..8 times kv_heads");
  const StaticLayout lay = static_layout(batch, q_heads, kv_heads, head_dim);
  if (lay.total > kStaticScratchBytes)
    return fail(MK_ERR_WORKSPACE,
                "mk_kv_attention_static: batch %d x %d query heads x head_dim %d needs %zu bytes of scratch, the static "
                "array holds %zu; use mk_kv_attention with a caller workspace", batch, q_heads, head_dim, lay.total,
                kStaticScratchBytes);
  if (reinterpret_cast<uintptr_t>(key_cache) % 16 || reinterpret_cast<uintptr_t>(value_cache) % 16)
    return fail(MK_ERR_ALIGNMENT, "mk_kv_attention_static: caches must be 16-byte aligned");
  int current = -1;
  MK_CUDA(cudaGetDevice(&current));
  if (current != device)
    return fail(MK_ERR_INVALID, "mk_kv_attention_static: device %d is not the current device (%d)", device, current);
  StaticSlot& slot = g_static_slots[device];
  std::lock_guard<std::mutex> guard(slot.lock);
  if (!slot.ready) {
    if (int e = static_setup(slot, device, static_cast<cudaStream_t>(stream))) return e;
  }
  // A handle on the stack (no device memory of its own) lets the shared parameter and
  // launch helpers serve this entry point unchanged.
  mk_handle_s view;
  memset(&view.cfg, 0, sizeof(view.cfg));
  view.cfg.hidden = q_heads * head_dim; view.cfg.layers = 1; view.cfg.q_heads = q_heads; view.cfg.kv_heads = kv_heads;
  view.cfg.head_dim = head_dim; view.cfg.intermediate = 64; view.cfg.vocab = 64; view.cfg.rms_eps = 1e-5f;
  view.cfg.rope_style = MK_ROPE_HF; view.cfg.max_tokens = batch; view.cfg.max_positions = capacity;
  view.cfg.engine = MK_ENGINE_TCGEN05;
  view.device = device; view.grid = slot.grid; view.ws = slot.base;
  view.cv = Carve{};
  view.cv.ctrl = lay.ctrl; view.cv.att_xch = lay.att_xch; view.cv.att_part = lay.att_part; view.cv.total = lay.total;
  view.bound = false;
  memset(&view.weights, 0, sizeof(view.weights));
  view.epoch = slot.epoch; view.att_epoch = slot.att_epoch; view.launches = slot.launches;
  view.timeout_cycles = slot.timeout_cycles;
  view.att_scale = static_cast<float>(std::pow(static_cast<double>(head_dim), -0.5));
  view.fma_ok = false; view.small_ll = false; view.row_ok = false; view.trace = nullptr; view.trace_cap = 0;
  view.mirror = nullptr; view.use3d = false;
  view.tp_epoch = 0; view.tp_bound = false;
  for (int r = 0; r < kMaxTp; ++r) view.tp_peer[r] = nullptr;
  if (int e = attention_fits(&view, capacity, "mk_kv_attention_static")) return e;
  KParams p;
  base_params(&view, p);
  p.mode = MODE_KVATT; p.m = batch; p.batch = batch; p.seq = 1; p.capacity = capacity;
  p.n_gemm = 0; p.nbar = 1;
  p.op_q = static_cast<const bf16*>(query); p.op_k = static_cast<const bf16*>(key); p.op_v = static_cast<const bf16*>(value);
  p.op_out = static_cast<bf16*>(output);
  p.kc[0] = key_cache; p.vc[0] = value_cache; p.len[0] = valid_length;
  if (int e = launch(&view, p, stream, 1)) return e;
  slot.epoch = view.epoch; slot.att_epoch = view.att_epoch; slot.launches = view.launches;
  return MK_OK;
}

}  // extern "C"
