// The persistent decoder megakernel for sm_100a: one cooperative launch runs a
// whole Llama/Qwen2-style decoder step (decode or prompt pass).
//
// Roles inside each CTA (one CTA per SM, 224 threads):
//   warp 0      weight producer: walks the static schedule of every projection
//               phase of the launch and streams this CTA's weight tiles through
//               a ring of TMA-filled shared-memory slots.  Weights never depend
//               on a barrier, so the stream runs ahead across phases and layers.
//   warp 6      activation producer: the token operand of a projection is a
//               bf16 matrix in global memory (normalised rows, attention output,
//               SiLU*up); once the workers signal that it is complete, this warp
//               streams its K chunks through a second ring with TMA, entry for
//               entry in step with the weight ring.  No thread copies operands.
//   warp 1      MMA issuer: tcgen05.mma with the weight tile as the M operand
//               and 16, 32 or 64 tokens as the N operand (the "swapAB"
//               orientation), fp32 accumulators in TMEM, one commit per ring
//               entry (an entry carries up to four 64-element K chunks).
//   warps 2-5   workers: RMSNorm as a distributed pass over token rows, the
//               epilogues out of TMEM (bias, residual add, SiLU*up, partial
//               sums), the attention phases (RoPE, KV append, split-context
//               softmax attention) and the grid barriers.
//
// Work split: the output rows of a projection phase are cut into tiles of
// `rows` rows (a multiple of 8), chosen on the host so the tile count is just
// under a multiple of the CTA count.  A CTA runs each of its tiles over the
// whole reduction length into one TMEM accumulator: a single fp32 chain per
// output, results do not depend on timing.  Only `rows` rows of the 128-row
// MMA tile hold weights; the tensor core computes the rest on stale bytes and
// the epilogue ignores them.  Launches of more than 64 tokens walk token tiles
// inside each weight tile, so the repeated passes over a tile come from L2.
//
// Every device wait is bounded: a wait that runs out records where in the
// status block, raises the abort flag that all other waits poll, and the CTA
// leaves through the common exit (drain TMA, free TMEM).  Nothing traps.
#pragma once
#include "megakernel.cuh"
#include "ptx.cuh"

namespace mk {

struct SmemMisc {
  uint64_t full[kChunkBars];
  uint64_t empty[kChunkBars];
  uint64_t accfull[2];
  uint64_t accempty[2];
  uint32_t tmem_base;
  int wabort;   // sticky: a worker thread gave up a wait
  int bad;      // prologue validation result
  int flag;
  int trace_n;  // events this CTA has recorded
  int trace_on; // copies of launch parameters the phases read often (a parameter read through the context costs two dependent loads)
  int n_gemm;
  uint32_t epoch;
  const GemmPhase* phases;
  float sred[kSplitTokens][8];   // small-launch kernel: per-token cross-warp sums
  long long pos_s[kSplitTokens]; // small-launch kernel: validated positions
  int len_s[MK_MAX_LAYERS];      // small-launch kernel: valid lengths before this call
  uint8_t qstart[kChunkBars];  // producer: first ring granule of each entry in flight (by sequence % kChunkBars)
  uint8_t qgran[kChunkBars];   // producer: granules of that entry
  GemmPhase phase[2];  // worker-side copies of the current / next projection phase
};
static_assert(sizeof(SmemMisc) <= kMiscBytes, "misc shared block too large");
static_assert(kRingGranules < 256, "ring positions are kept in bytes");

// Decode attention's cache stages in the weight ring (see attention_decode).
#ifndef MK_DEC_STAGES
#define MK_DEC_STAGES 3
#endif
#ifndef MK_DEC_TILE_KB
#define MK_DEC_TILE_KB 32
#endif
constexpr int kDecStages = MK_DEC_STAGES;
constexpr int kDecScratchBytes = 13 * 1024;  // q [8][128] fp32 and bf16, value partial sums [1024] fp32, new keys/values [2][512] bf16, statistics
constexpr int kDecTileBytes = MK_DEC_TILE_KB * 1024;  // one stage

// Tensor engine only: the activation ring's barriers and bookkeeping (behind SmemMisc).
struct SmemMiscTc {
  uint64_t bfull[kChunkBars];
  uint64_t bempty[kChunkBars];
  uint8_t bstart[kChunkBars];
  uint8_t bgran[kChunkBars];
  int b_ready;  // projection phases whose activation operand is complete in global memory (workers -> activation producer)
  int a_ready;  // gated projection phases whose weights may be fetched: the workers no longer use the ring (workers -> weight producer)
  int kv_seq;   // cache tiles fetched by TMA so far in this launch (stage and barrier parity of the next one)
  uint64_t kvfull[8];   // cache stages: the copy has landed
  uint64_t kvempty[8];  // cache stages: every worker warp is done with the tile
  // The cache stream of one attention unit, asked for by the workers and issued by the (otherwise idle) weight
  // producer: K tiles 0 .. nt-1, then V tiles 0 .. nt-1, of `tile_keys` positions from position t0 on.
  int kv_req;           // units asked for so far in this launch (workers -> weight producer)
  struct KvRequest {
    const CUtensorMap *kmap, *vmap;
    int t0, nt, tile_keys, chunk0, b, gtile;
    uint32_t stage_bytes;
  } kvr;
};
static_assert(sizeof(SmemMiscTc) <= kMiscTcBytes, "tensor-engine misc block too large");
static_assert(kBBytes / kGranule < 256, "activation ring positions are kept in bytes");

struct Ctx {
  const KParams* p;
  Control* ctrl;
  SmemMisc* misc;
  SmemMiscTc* tc;   // null in the small-launch kernel
  uint8_t* smem_a;
  uint8_t* smem_b;
  long long deadline;
  int cta, grid;
};

// Worker-side running state across the phases of one launch.
struct WorkerState {
  uint32_t tiles;        // accumulator buffers consumed so far
  uint32_t passed;       // grid barriers passed
};

// ---------------------------------------------------------------------------
// bounded waits

// Waits between CTAs or GPUs (grid barrier, attention exchange, tensor-parallel flag) give up at the
// deadline; waits inside a CTA's own pipeline (ring slots, accumulators) an eighth of the limit later,
// so that when a peer is late the status names the wait on the peer, not a thread starved behind it.
__device__ __forceinline__ bool give_up(const Ctx& cx, int site, int detail) {
  if (ld_relaxed_u32(&cx.ctrl->abort) != 0) return true;
  const bool internal = site == SITE_PRODUCER_EMPTY || site == SITE_MMA_FULL || site == SITE_MMA_B || site == SITE_MMA_ACC ||
                        site == SITE_EPI_ACC || site == SITE_B_EMPTY || site == SITE_KV_TILE;
  if (clock64() > cx.deadline + (internal ? (cx.p->timeout_cycles >> 3) : 0)) {
    if (atomicCAS(&cx.ctrl->status, 0, static_cast<int>(MK_STATUS_TIMEOUT)) == 0) {
      cx.ctrl->where = site;
      cx.ctrl->cta = cx.cta;
      cx.ctrl->detail = detail;
      if (cx.p->status_mirror) *cx.p->status_mirror = static_cast<int>(MK_STATUS_TIMEOUT);
    }
    atomicExch(&cx.ctrl->abort, 1u);
    __threadfence();
    return true;
  }
  return false;
}

// Optional per-CTA event trace (worker thread 0 only): what the reference's
// MEGABAKE_PHASE_TIMER stamps give (src/megabake/runtime.py:27-46).
__device__ __noinline__ void trace_event_record(const Ctx& cx, int code) {
  const int n = cx.misc->trace_n;
  if (n >= cx.p->trace_cap) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  cx.p->trace[static_cast<size_t>(cx.cta) * cx.p->trace_cap + n] =
      (static_cast<unsigned long long>(code) << 56) | (t & 0x00FFFFFFFFFFFFFFull);
  cx.misc->trace_n = n + 1;
}
// The test is inline, the recording out of line: with tracing off an event costs a compare.
__device__ __forceinline__ void trace_event(const Ctx& cx, int wtid, int code) {
  if (wtid == 0 && cx.misc->trace_on != 0) trace_event_record(cx, code);
}

__device__ __forceinline__ bool wait_mbar(const Ctx& cx, uint32_t bar, uint32_t parity, int site, int detail) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (++spins > 8) __nanosleep(64);  // a long wait must not steal issue slots from the warps that share this scheduler
    if ((spins & 255u) == 0 && give_up(cx, site, detail)) return false;
  }
  return true;
}

// Same wait, adding the cycles it took to `cycles` (profiling of the single-thread roles).
__device__ __forceinline__ bool wait_mbar_timed(const Ctx& cx, uint32_t bar, uint32_t parity, int site, int detail,
                                                long long& cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  const bool ok = wait_mbar(cx, bar, parity, site, detail);
  cycles += clock64() - t0;
  return ok;
}

// Worker-uniform decision: true only if no worker thread has given up.
__device__ __forceinline__ bool workers_ok(const Ctx& cx, bool ok) {
  if (!ok) cx.misc->wabort = 1;
  named_bar_sync(1, kWorkers);
  return *reinterpret_cast<volatile int*>(&cx.misc->wabort) == 0;
}

// Monotonic-counter grid barrier over the worker warps of every CTA: one
// release-add to arrive, relaxed polling, one fence once the count is reached.
__device__ bool grid_barrier(const Ctx& cx, WorkerState& ws, int wtid) {
  fence_proxy_async_all();  // what this thread stored may be the next phase's TMA-loaded operand in another CTA
  named_bar_sync(1, kWorkers);
  ws.passed += 1;
  if (wtid == 0) {
    red_release_add_u32(&cx.ctrl->barrier, 1u);
    const uint32_t target = cx.p->epoch + ws.passed * static_cast<uint32_t>(cx.grid);
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_relaxed_u32(&cx.ctrl->barrier) - target) < 0) {
      if ((++spins & 255u) == 0 && give_up(cx, SITE_GRID_BARRIER, static_cast<int>(ws.passed))) {
        cx.misc->wabort = 1;
        break;
      }
    }
    __threadfence();
  }
  named_bar_sync(1, kWorkers);
  trace_event(cx, wtid, EV_BARRIER_DONE);
  return *reinterpret_cast<volatile int*>(&cx.misc->wabort) == 0;
}

// ---------------------------------------------------------------------------
// schedule helpers shared by the three roles

__device__ __forceinline__ void tile_origin(const GemmPhase* ph, int tile, int& seg, int& row0) {
  seg = 0;
  if (ph->nacc == 1) {
    while (seg + 1 < ph->nseg && tile >= ph->tile_start[seg + 1]) ++seg;
  }
  row0 = (tile - ph->tile_start[seg]) * ph->rows;
}

// Every CTA walks its K slice from a different starting chunk (and wraps), so
// that at any moment the grid's loads spread over all of a weight row's
// 128-byte columns.  Slices whose activation operand is streamed in batches of
// kBHalf chunks rotate by whole batches.
__device__ __forceinline__ int k_rotation(int cta, int grid, int kslice) {
  if (kslice <= kBSlots) return static_cast<int>((static_cast<long long>(cta) * kslice) / grid);
  const int batches = (kslice + kBHalf - 1) / kBHalf;
  return static_cast<int>((static_cast<long long>(cta) * batches) / grid);  // in batches
}

// Phase gp of the launch: a row of the phase table in global memory, or, for a stand-alone projection, the
// descriptor that came with the kernel parameters.
__device__ __forceinline__ const GemmPhase* phase_at(const KParams& p, int gp) {
  return p.mode == MODE_LINEAR ? &p.linear_phase : p.phases + gp;
}

// Tokens per MMA (UMMA N) for a launch of m tokens: the smallest of 16, 32, 64, 128 that holds them, 128 beyond
// (an MMA of 128 columns costs 64 issue cycles where two of 64 cost 92, and a weight tile is walked half as often).
__device__ __forceinline__ int token_tile(int m) { return m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128)); }
__device__ __forceinline__ int token_tile_index(int m) { return m <= 16 ? 0 : (m <= 32 ? 1 : (m <= 64 ? 2 : 3)); }

// Every CTA walks its K range from a different starting entry (and wraps), so that at any moment the
// grid's loads spread over all of a weight row's 128-byte columns.
__device__ __forceinline__ int group_rotation(int cta, int grid, int groups) {
  return static_cast<int>((static_cast<long long>(cta) * groups) / grid);
}

// A ring of 1 KiB granules handed out in FIFO order; an entry never wraps.  Entries are consumed in
// issue order, so space is reclaimed by retiring the oldest entry in flight (waiting for its `empty`
// barrier) until the wanted granules are free.  One instance per producer.
struct RingCursor {
  int head, seq, oldest;
};

__device__ __forceinline__ bool ring_claim(const Ctx& cx, RingCursor& rc, int total, int gran, uint64_t* empty,
                                           uint8_t* qstart, uint8_t* qgran, int site, int gp, int& start) {
  auto retire = [&]() -> bool {
    const bool done = wait_mbar(cx, smem_u32(&empty[rc.oldest % kChunkBars]), (rc.oldest / kChunkBars) & 1, site, gp);
    ++rc.oldest;
    return done;
  };
  auto reclaim = [&](int lo, int hi) -> bool {
    while (rc.oldest < rc.seq) {
      const int os = qstart[rc.oldest % kChunkBars], oe = os + qgran[rc.oldest % kChunkBars];
      if (!(os < hi && lo < oe)) break;
      if (!retire()) return false;
    }
    return true;
  };
  if (rc.head + gran > total) {  // the tail fragment is skipped: free it too, then wrap
    if (!reclaim(rc.head, total)) return false;
    rc.head = 0;
  }
  start = rc.head;
  rc.head += gran;
  if (!reclaim(start, start + gran)) return false;
  if (rc.seq - rc.oldest >= kChunkBars && !retire()) return false;  // barrier pair reuse
  qstart[rc.seq % kChunkBars] = static_cast<uint8_t>(start);
  qgran[rc.seq % kChunkBars] = static_cast<uint8_t>(gran);
  return true;
}

// Leaving early: every copy already issued must land before the CTA exits.
__device__ __forceinline__ void ring_drain(const RingCursor& rc, uint64_t* full) {
  for (int i = max(0, rc.seq - kChunkBars); i < rc.seq; ++i) {
    const uint32_t bar = smem_u32(&full[i % kChunkBars]);
    for (uint32_t spins = 0; spins < (1u << 22); ++spins) {
      if (mbar_try_wait(bar, (i / kChunkBars) & 1)) break;
    }
  }
}

// ---------------------------------------------------------------------------
// warp 0: weight producer
//
// An entry of the weight ring holds `kb` consecutive 64-element K chunks of a tile's rows, for each
// accumulator matrix of the phase (gate and up side by side):
//     [matrix 0: kb x (rows x 128 B, 128-byte swizzled)][matrix 1: ...]
// One three-dimensional TMA box (64 elements, rows, kb chunks) brings a matrix's share, so a copy
// carries 14-32 KB where a single chunk of a 56-row tile would carry 7 KB.
// The cache stream of the attention unit the workers have posted (see attention_decode_stream): one tiled copy
// per stage as soon as every worker warp has released the stage's previous tile.
__device__ __noinline__ bool serve_cache_stream(const Ctx& cx) {
  SmemMiscTc* tc = cx.tc;
  __threadfence_block();
  const volatile SmemMiscTc::KvRequest* r = &tc->kvr;
  const CUtensorMap* const kmap = r->kmap;
  const CUtensorMap* const vmap = r->vmap;
  const int t0 = r->t0, nt = r->nt, tile_keys = r->tile_keys, chunk0 = r->chunk0, b = r->b, gtile = r->gtile;
  const uint32_t stage_bytes = r->stage_bytes;
  const uint32_t tiles = smem_u32(cx.smem_a);
  const uint32_t kvfull0 = smem_u32(&tc->kvfull[0]), kvempty0 = smem_u32(&tc->kvempty[0]);
  const uint64_t policy = l2_policy_evict_first();
  int stage = gtile % kDecStages, use = gtile / kDecStages;  // earlier uses of `stage` in this launch
#pragma unroll 1
  for (int s = 0; s < 2 * nt; ++s) {
    if (use > 0 && !wait_mbar(cx, kvempty0 + stage * 8u, (use - 1) & 1, SITE_KV_TILE, -s)) return false;
    const uint32_t bar = kvfull0 + stage * 8u;
    mbar_expect_tx(bar, stage_bytes);
    const int t = (s < nt) ? s : s - nt;
    tma_load_4d(tiles + stage * stage_bytes, (s < nt) ? kmap : vmap, 0, t0 + t * tile_keys, chunk0, b, bar, policy);
    if (++stage == kDecStages) {
      stage = 0;
      ++use;
    }
  }
  return true;
}

__device__ __noinline__ void producer_loop(const Ctx& cx) {
  const KParams& p = *cx.p;
  int kv_served = 0;
  const uint64_t policy = p.stream_once ? l2_policy_evict_first() : l2_policy_evict_normal();
  const int ntok = token_tile(p.m);
  const int ntt = (p.m + ntok - 1) / ntok;
  SmemMisc* misc = cx.misc;
  RingCursor rc;
  rc.head = 0; rc.seq = 0; rc.oldest = 0;
  bool ok = true;
  for (int gp = 0; gp < p.n_gemm && ok; ++gp) {
    const GemmPhase* ph = phase_at(p, gp);
    const int nacc = ph->nacc, gran = ph->gran, nunits = ph->nunits, ksplit = ph->ksplit, kslice = ph->kslice, kb = ph->kb;
    const uint32_t matrix_bytes = static_cast<uint32_t>(ph->rows) * 128u * static_cast<uint32_t>(kb);
    const int groups = kslice / kb;
    const int rot = group_rotation(cx.cta, cx.grid, groups);
    const int map3d = ph->map3d;
    // descriptor pointers in registers: every barrier wait below is a compiler barrier for memory, and a
    // field read again behind it costs this one thread a round trip to L2 per copy
    const bool linear = p.mode == MODE_LINEAR;
    const CUtensorMap* const m0 = linear ? &p.linear_wmap : ph->tmap[0];
    const CUtensorMap* const m1 = linear ? &p.linear_wmap : ph->tmap[1];
    const CUtensorMap* const m2 = linear ? &p.linear_wmap : ph->tmap[2];
    const int nseg = ph->nseg, rows = ph->rows, ts1 = ph->tile_start[1], ts2 = ph->tile_start[2];
    if (ph->gate) {  // the attention phase before this one streams cache tiles through the ring
      uint32_t spins = 0;
      while (*reinterpret_cast<volatile int*>(&cx.tc->a_ready) <= gp) {
        if (*reinterpret_cast<volatile int*>(&cx.tc->kv_req) != kv_served) {  // an attention unit wants its cache tiles
          if (!serve_cache_stream(cx)) {
            ok = false;
            break;
          }
          ++kv_served;
          continue;
        }
        __nanosleep(64);
        if ((++spins & 255u) == 0 && give_up(cx, SITE_PRODUCER_EMPTY, -gp)) {
          ok = false;
          break;
        }
      }
      if (!ok) break;
    }
    for (int unit = cx.cta; unit < nunits && ok; unit += cx.grid) {
      const int tile = unit / ksplit, slice = unit - tile * ksplit;
      int seg = 0;  // tile_origin() on the private copies
      if (nacc == 1) {
        if (nseg > 1 && tile >= ts1) seg = 1;
        if (nseg > 2 && tile >= ts2) seg = 2;
      }
      const int row0 = (tile - (seg == 0 ? 0 : (seg == 1 ? ts1 : ts2))) * rows;
      const CUtensorMap* const map_seg = seg == 0 ? m0 : (seg == 1 ? m1 : m2);
      const int kbase = slice * kslice;
      for (int tt = 0; tt < ntt && ok; ++tt) {
        int g = rot;
        for (int i = 0; i < groups; ++i) {
          int start;
          if (!ring_claim(cx, rc, kRingGranules, gran, misc->empty, misc->qstart, misc->qgran, SITE_PRODUCER_EMPTY, gp, start)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&misc->full[rc.seq % kChunkBars]);
          const uint32_t dst = smem_u32(cx.smem_a + start * kGranule);
          mbar_expect_tx(full, matrix_bytes * static_cast<uint32_t>(nacc));
          for (int a = 0; a < nacc; ++a) {
            const CUtensorMap* map = nacc == 2 ? (a ? m1 : m0) : map_seg;
            if (map3d) {
              tma_load_3d(dst + a * matrix_bytes, map, 0, row0, kbase + g * kb, full, policy);
            } else {
              for (int c = 0; c < kb; ++c)
                tma_load_2d(dst + a * matrix_bytes + c * (matrix_bytes / kb), map, (kbase + g * kb + c) * kChunkK, row0, full, policy);
            }
          }
          ++rc.seq;
          g = (g + 1 == groups) ? 0 : g + 1;
        }
      }
    }
  }
  if (!ok) ring_drain(rc, misc->full);
}

// ---------------------------------------------------------------------------
// warp 6: activation producer
//
// The token operand of phase gp is rows [tt * ntok, +ntok) x K of a bf16 matrix in global memory.
// Its entries mirror the weight ring's one for one (same unit, token tile and K group order): entry
// = kb boxes of (64 elements x ntok tokens), 128-byte swizzled, rows past the matrix read as zero.
// The matrix is written by other CTAs during the preceding phase, so this warp starts a phase only
// after the workers, having passed the grid barrier, publish it in `b_ready`.
__device__ __noinline__ void activation_producer_loop(const Ctx& cx) {
  const KParams& p = *cx.p;
  const uint64_t policy = l2_policy_evict_normal();
  const int ntok = token_tile(p.m), tile_index = token_tile_index(p.m);
  const int ntt = (p.m + ntok - 1) / ntok;
  SmemMiscTc* tc = cx.tc;
  RingCursor rc;
  rc.head = 0; rc.seq = 0; rc.oldest = 0;
  bool ok = true;
  for (int gp = 0; gp < p.n_gemm && ok; ++gp) {
    const GemmPhase* ph = phase_at(p, gp);
    const int nunits = ph->nunits, ksplit = ph->ksplit, kslice = ph->kslice, kb = ph->kb;
    if (cx.cta >= nunits) continue;
    {  // wait for the operand of this phase
      uint32_t spins = 0;
      while (*reinterpret_cast<volatile int*>(&tc->b_ready) <= gp) {
        __nanosleep(64);
        if ((++spins & 255u) == 0 && give_up(cx, SITE_MMA_B, gp)) {
          ok = false;
          break;
        }
      }
      if (!ok) break;
      fence_proxy_async_all();  // generic-proxy stores of the operand (acquired through the barrier) before async-proxy reads
    }
    const CUtensorMap* map = p.mode == MODE_LINEAR ? &p.linear_xmap : ph->bmap[tile_index];
    const int groups = kslice / kb;
    const int rot = group_rotation(cx.cta, cx.grid, groups);
    const int gran = kb * ntok / 8;
    const uint32_t chunk_bytes = static_cast<uint32_t>(ntok) * 128u;
    for (int unit = cx.cta; unit < nunits && ok; unit += cx.grid) {
      const int slice = unit % ksplit;
      const int kbase = slice * kslice;
      for (int tt = 0; tt < ntt && ok; ++tt) {
        int g = rot;
        for (int i = 0; i < groups; ++i) {
          int start;
          if (!ring_claim(cx, rc, kBBytes / kGranule, gran, tc->bempty, tc->bstart, tc->bgran, SITE_B_EMPTY, gp, start)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&tc->bfull[rc.seq % kChunkBars]);
          const uint32_t dst = smem_u32(cx.smem_b + start * kGranule);
          mbar_expect_tx(full, chunk_bytes * static_cast<uint32_t>(kb));
          for (int c = 0; c < kb; ++c)
            tma_load_2d(dst + c * chunk_bytes, map, (kbase + g * kb + c) * kChunkK, tt * ntok, full, policy);
          ++rc.seq;
          g = (g + 1 == groups) ? 0 : g + 1;
        }
      }
    }
  }
  if (!ok) ring_drain(rc, tc->bfull);
}

// ---------------------------------------------------------------------------
// warp 1: MMA issuer

__device__ __noinline__ void mma_loop(const Ctx& cx) {
  const KParams& p = *cx.p;
  const int ntok = token_tile(p.m);
  const int ntt = (p.m + ntok - 1) / ntok;
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&cx.misc->tmem_base);
  // A tile of at most 64 weight rows is issued as an M = 64 MMA: in the running kernel an MMA's time is the read
  // of its weight operand from shared memory (128 rows x 32 B), and half the rows are read in half the time.
  const uint32_t idesc128 = umma_idesc_bf16(kTileRows, ntok), idesc64 = umma_idesc_bf16(64, ntok);
  const uint64_t desc_base = umma_desc_sw128(0);
  const uint32_t desc_lo = static_cast<uint32_t>(desc_base), desc_hi = static_cast<uint32_t>(desc_base >> 32);
  const uint32_t b_step = (static_cast<uint32_t>(ntok) * 128u) >> 4;
  const uint32_t ring_base = smem_u32(cx.smem_a), b_base = smem_u32(cx.smem_b);
  SmemMisc* misc = cx.misc;
  SmemMiscTc* tc = cx.tc;
  int seq = 0;
  uint32_t q = 0;
  for (int gp = 0; gp < p.n_gemm; ++gp) {
    const GemmPhase* ph = phase_at(p, gp);
    const int nacc = ph->nacc, nunits = ph->nunits, kslice = ph->kslice, kb = ph->kb;
    const uint32_t a_step = (static_cast<uint32_t>(ph->rows) * 128u) >> 4;
    const uint32_t idesc = ph->rows <= 64 ? idesc64 : idesc128;
    const int groups = kslice / kb;
    if (cx.cta >= nunits) continue;
    for (int unit = cx.cta; unit < nunits; unit += cx.grid) {
      for (int tt = 0; tt < ntt; ++tt) {
        const uint32_t buf = q & 1u;
        if (!wait_mbar(cx, smem_u32(&misc->accempty[buf]), ((q >> 1) & 1u) ^ 1u, SITE_MMA_ACC, gp)) return;
        tc_fence_after();
        uint32_t accumulate = 0;
        const uint32_t d0 = tmem + buf * 2u * kMaxTok;
        for (int i = 0; i < groups; ++i) {
          const uint32_t parity = (seq / kChunkBars) & 1;
          if (!wait_mbar(cx, smem_u32(&misc->full[seq % kChunkBars]), parity, SITE_MMA_FULL, gp)) return;
          if (!wait_mbar(cx, smem_u32(&tc->bfull[seq % kChunkBars]), parity, SITE_MMA_B, gp)) return;
          tc_fence_after();
          // the producers recorded where they put this entry before they issued its copies
          const uint32_t a_addr = ring_base + static_cast<uint32_t>(misc->qstart[seq % kChunkBars]) * kGranule;
          const uint32_t b_addr = b_base + static_cast<uint32_t>(tc->bstart[seq % kChunkBars]) * kGranule;
          // descriptor low words of the entry's first chunk; a chunk further on is a constant further on
          uint32_t a_lo = desc_lo + (a_addr >> 4), b_lo = desc_lo + (b_addr >> 4);
          if (nacc == 1) {
#pragma unroll 1
            for (int c = 0; c < kb; ++c) {
              umma_bf16_chunk(d0, a_lo, b_lo, desc_hi, idesc, accumulate);
              accumulate = 1u;
              a_lo += a_step;
              b_lo += b_step;
            }
          } else {  // gate and up: the second matrix's chunks follow the first matrix's in the entry
            const uint32_t second = static_cast<uint32_t>(kb) * a_step;
#pragma unroll 1
            for (int c = 0; c < kb; ++c) {
              umma_bf16_chunk(d0, a_lo, b_lo, desc_hi, idesc, accumulate);
              umma_bf16_chunk(d0 + kMaxTok, a_lo + second, b_lo, desc_hi, idesc, accumulate);
              accumulate = 1u;
              a_lo += a_step;
              b_lo += b_step;
            }
          }
          umma_commit(smem_u32(&misc->empty[seq % kChunkBars]));
          umma_commit(smem_u32(&tc->bempty[seq % kChunkBars]));
          ++seq;
        }
        umma_commit(smem_u32(&misc->accfull[buf]));
        ++q;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// workers: helpers for rows of activations

__device__ __forceinline__ const bf16* activation_row(const KParams& p, const GemmPhase* ph, int token) {
  if (ph->gather) {
    long long id = p.ids[token];
    if (id < 0 || id >= p.embed_rows) id = 0;  // reported by the prologue; never dereference out of range
    return p.embed + id * p.hidden;
  }
  return ph->src + static_cast<size_t>(token) * ph->src_ld;
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

// bf16 -> fp32 is a 16-bit shift; keeping it in integer registers avoids taking addresses.
__device__ __forceinline__ void unpack8(const uint4 u, float* f) {
  f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xFFFF0000u);
  f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xFFFF0000u);
  f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xFFFF0000u);
  f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xFFFF0000u);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return static_cast<uint32_t>(__bfloat16_as_ushort(h.x)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h.y)) << 16);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}

// Normalise one 8-element vector: w * bf16(x * rinv), the two roundings of the
// Hugging Face RMSNorm.
// The second product is taken on bf16 pairs: the product of two bf16 values is exact in fp32, so
// the packed multiply's single rounding equals rounding the fp32 product (4 instructions for 8 values;
// the staging loops are bound by the instruction rate of the four worker warps).
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint4 normalise_vec(const uint4 xu, const uint4 wu, float r) {
  float x[8];
  unpack8(xu, x);
  return make_uint4(mul_bf16x2(wu.x, pack2(x[0] * r, x[1] * r)), mul_bf16x2(wu.y, pack2(x[2] * r, x[3] * r)),
                    mul_bf16x2(wu.z, pack2(x[4] * r, x[5] * r)), mul_bf16x2(wu.w, pack2(x[6] * r, x[7] * r)));
}

// Attention output for 8 consecutive columns of one token: the bf16 buffer when
// the context was not split, else the chunk partials summed in chunk order and
// rounded once.
__device__ __forceinline__ uint4 attention_vec(const KParams& p, int token, int col, int nch) {
  if (nch <= 1) return __ldcg(reinterpret_cast<const uint4*>(p.attn + static_cast<size_t>(token) * p.q_heads * p.head_dim + col));
  const int head = col / p.head_dim, d = col - head * p.head_dim;
  const float4* part = reinterpret_cast<const float4*>(
      p.att_part + (static_cast<size_t>(token) * p.q_heads + head) * kMaxChunks * p.head_dim + d);
  const int stride = p.head_dim / 4;  // float4s per chunk
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int c0 = 0; c0 < nch; c0 += 4) {
    float4 lo[4], hi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (c0 + i < nch) {
        lo[i] = __ldcg(part + (c0 + i) * stride);
        hi[i] = __ldcg(part + (c0 + i) * stride + 1);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (c0 + i < nch) {
        acc[0] += lo[i].x; acc[1] += lo[i].y; acc[2] += lo[i].z; acc[3] += lo[i].w;
        acc[4] += hi[i].x; acc[5] += hi[i].y; acc[6] += hi[i].z; acc[7] += hi[i].w;
      }
    }
  }
  return pack8(acc);
}

// ---------------------------------------------------------------------------
// workers: epilogues

__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ float ldcg_bf16(const bf16* ptr) {
  return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(ptr))));
}

// Values an epilogue adds to the accumulators; loaded before the accumulator
// wait so their latency hides behind the MMA: the residual stream (per token)
// or the bias (one value).
template <int NT>
__device__ __forceinline__ void epilogue_prefetch(const Ctx& cx, const GemmPhase* ph, int seg, int n, int t0, int mt,
                                                  float* pre) {
  if (ph->epi == EPI_RESIDUAL) {
#pragma unroll
    for (int t = 0; t < NT; ++t)
      if (t < mt) pre[t] = ldcg_bf16(ph->dst + static_cast<size_t>(t0 + t) * ph->dst_ld + n);
  } else if (ph->epi == EPI_STORE) {
    pre[0] = ph->bias[seg] ? ldg_bf16(ph->bias[seg] + n) : 0.f;
  }
}

// EPI_PARTIAL: this unit's fp32 sums over its K slice, for the next phase to add up.
template <int NT>
__device__ __forceinline__ void store_partial(const Ctx& cx, const GemmPhase* ph, int slice, int n, const float* v,
                                              int t0, int mt) {
#pragma unroll
  for (int t = 0; t < NT; ++t)
    if (t < mt) __stcg(ph->partial + (static_cast<size_t>(slice) * cx.p->m + (t0 + t)) * ph->n[0] + n, v[t]);
}

// Where source rank `src`'s partial sums of half `half` live in rank `peer`'s exchange buffer.
__device__ __forceinline__ float* tp_slot(const KParams& p, int peer, int half, int src) {
  return reinterpret_cast<float*>(p.tp_peer[peer] + kTpFlagBytes) +
         (static_cast<size_t>(half) * p.tp_size + src) * p.m * p.hidden;
}

// EPI_TP: this rank's fp32 sums over its share of the reduction length go, unrounded, into the
// slot of this rank in every rank's exchange buffer (plain peer stores over NVLink; the local
// rank is one of them).  The all-reduce is finished by tp_allreduce once every rank has stored.
template <int NT>
__device__ __forceinline__ void store_tp_partial(const Ctx& cx, const GemmPhase* ph, int n, const float* v, int t0, int mt) {
  const KParams& p = *cx.p;
  for (int peer = 0; peer < p.tp_size; ++peer) {
    float* dst = tp_slot(p, peer, ph->tp_buf, p.tp_rank) + n;
#pragma unroll
    for (int t = 0; t < NT; ++t)
      if (t < mt) dst[static_cast<size_t>(t0 + t) * p.hidden] = v[t];
  }
}

// Finish output row n of matrix `seg` for the tokens of the tile.
template <int NT>
__device__ __forceinline__ void apply_epilogue(const Ctx& cx, const GemmPhase* ph, int seg, int n, float (*v)[NT],
                                               const float* pre, int t0, int mt) {
  const KParams& p = *cx.p;
  if (ph->epi == EPI_SILU) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (t < mt) {
        const float gate = bf16_round(v[0][t]);
        const float up = bf16_round(v[1][t]);
        const float act = bf16_round(silu(gate));
        ph->dst[static_cast<size_t>(t0 + t) * ph->dst_ld + n] = __float2bfloat16_rn(act * up);
      }
    }
    return;
  }
  bf16* dst = ph->to_logits ? p.logits : ph->dst;
  const size_t col = static_cast<size_t>(ph->out_col[seg]) + n;
  if (ph->epi == EPI_STORE) {
#pragma unroll
    for (int t = 0; t < NT; ++t)
      if (t < mt) dst[static_cast<size_t>(t0 + t) * ph->dst_ld + col] = __float2bfloat16_rn(v[0][t] + pre[0]);
  } else {  // EPI_RESIDUAL: hidden += bf16(projection), in place
#pragma unroll
    for (int t = 0; t < NT; ++t)
      if (t < mt) dst[static_cast<size_t>(t0 + t) * ph->dst_ld + col] = __float2bfloat16_rn(pre[t] + bf16_round(v[0][t]));
  }
}

// Copy the next projection phase's descriptor into shared memory so that no
// worker pays a global round trip for it after the barrier.
__device__ __forceinline__ void prefetch_phase(const Ctx& cx, int gp, int wtid) {
  if (gp >= cx.p->n_gemm) return;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(phase_at(*cx.p, gp));
  uint32_t* dst = reinterpret_cast<uint32_t*>(&cx.misc->phase[gp & 1]);
  for (int i = wtid; i < static_cast<int>(sizeof(GemmPhase) / 4); i += kWorkers) dst[i] = __ldg(src + i);
}

// Projection phase on the tcgen05 engine, worker side: the epilogues.  The caller has made phase
// gp's descriptor visible in cx.misc->phase[gp & 1] and published the phase's operand (signal_operand).
// A warp may read TMEM lanes [32 * (warp index % 4), +32): thread (quadrant, lane) finishes weight row
// quadrant * 32 + lane of the tile, sixteen token columns at a time.
__device__ __noinline__ bool worker_gemm_tc(const Ctx& cx, int gp, WorkerState& ws, int wtid) {
  const int m = cx.p->m;  // read once: the waits below are compiler barriers for memory
  const GemmPhase* ph = &cx.misc->phase[gp & 1];
  const int ntok = token_tile(m);
  const int ntt = (m + ntok - 1) / ntok;
  const int nacc = ph->nacc, nunits = ph->nunits, rows = ph->rows, ksplit = ph->ksplit, epi = ph->epi;
  const uint32_t accfull0 = smem_u32(&cx.misc->accfull[0]), accempty0 = smem_u32(&cx.misc->accempty[0]);
  const int my_cta = cx.cta, grid = cx.grid;
  const int quad = ((wtid >> 5) + 2) & 3;  // TMEM lane quadrant this warp may read
  // M = 128: accumulator row r is TMEM lane r.  M = 64 (tiles of at most 64 rows): row r is lane 32 * (r / 16) + r % 16,
  // the upper half of every quadrant is unused.
  const bool m64 = rows <= 64;
  const int lane_id = wtid & 31;
  const int rloc = m64 ? (lane_id < 16 ? quad * 16 + lane_id : kTileRows) : quad * 32 + lane_id;
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&cx.misc->tmem_base);
  if (my_cta < nunits) {
    trace_event(cx, wtid, EV_PHASE_ENTER);
    for (int unit = my_cta; unit < nunits; unit += grid) {
      const int tile = unit / ksplit, slice = unit - tile * ksplit;
      int seg, row0;
      tile_origin(ph, tile, seg, row0);
      const int n = row0 + rloc;
      const bool valid = rloc < rows && n < ph->n[seg];
      for (int tt = 0; tt < ntt; ++tt) {
        const uint32_t buf = ws.tiles & 1u;
        bool ok = wait_mbar(cx, accfull0 + buf * 8u, (ws.tiles >> 1) & 1u, SITE_EPI_ACC, gp);
        ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
        if (unit == my_cta && tt == 0) trace_event(cx, wtid, EV_FIRST_ACC);
        tc_fence_after();
        const int tile_tokens = min(ntok, m - tt * ntok);
        // the two warps that share a TMEM lane quadrant take alternate groups of sixteen token columns
        for (int cg = (wtid >> 5) / 4; cg * kTok < tile_tokens; cg += kWorkerWarps / 4) {
          const int t0 = tt * ntok + cg * kTok;
          const int mt = min(kTok, m - t0);
          float pre[kTok];
          if (valid) epilogue_prefetch<kTok>(cx, ph, seg, n, t0, mt, pre);
          float v[2][kTok];
          if (ok && (m64 ? quad * 16 : quad * 32) < rows) {
            const uint32_t at = tmem + (static_cast<uint32_t>(quad * 32) << 16) + (buf * 2u) * kMaxTok + cg * kTok;
            tmem_ld16(at, v[0]);
            if (nacc == 2) tmem_ld16(at + kMaxTok, v[1]);
          }
          if (ok && valid) {
            if (epi == EPI_PARTIAL) store_partial<kTok>(cx, ph, slice, n, v[0], t0, mt);
            else if (epi == EPI_TP) store_tp_partial<kTok>(cx, ph, n, v[0], t0, mt);
            else apply_epilogue<kTok>(cx, ph, seg, n, v, pre, t0, mt);
          }
        }
        tc_fence_before();
        mbar_arrive(accempty0 + buf * 8u);
        ws.tiles += 1;
        if (!workers_ok(cx, ok)) return false;
      }
    }
    trace_event(cx, wtid, EV_PHASE_DONE);
  }
  if (ph->epi == EPI_TP) __threadfence_system();  // this thread's peer stores are performed before it arrives at the grid barrier
  prefetch_phase(cx, gp + 1, wtid);
  return true;
}

// Tell the activation producer that phase gp's operand is complete (called after the grid barrier
// that closes whatever wrote it; for the first phase of a stand-alone projection, at once).
__device__ __forceinline__ void signal_operand(const Ctx& cx, int gp, int wtid) {
  if (wtid == 0) *reinterpret_cast<volatile int*>(&cx.tc->b_ready) = gp + 1;
}

// One 8-element vector of the residual stream after the pending update (see norm_phase).
__device__ __forceinline__ uint4 residual_vec(const Ctx& cx, const GemmPhase* ph, int token, int v) {
  const KParams& p = *cx.p;
  const uint4 xu = __ldcg(reinterpret_cast<const uint4*>(activation_row(p, ph, token)) + v);
  if (ph->add_parts == 0) return xu;
  float f[8], acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  unpack8(xu, f);
  for (int s8 = 0; s8 < ph->add_parts; ++s8) {
    const float4* part = reinterpret_cast<const float4*>(ph->partial + (static_cast<size_t>(s8) * p.m + token) * ph->k) + v * 2;
    const float4 lo = __ldcg(part), hi = __ldcg(part + 1);
    acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
    acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = bf16_round(f[e] + bf16_round(acc[e]));
  return pack8(f);
}

// RMSNorm as a phase of its own, ahead of the projections that take normalised rows: one CTA of the
// grid per token row, every worker thread a few 8-element vectors of it, all of a thread's loads in
// flight together.  The row is the residual stream (or, in layer 0, the embedding row of the token
// id) plus, on the split-K table, the pending update x = residual + bf16(sum of the previous
// projection's fp32 K-slice partials, in slice order), which is written back as the new residual
// stream.  The normalised row, w * bf16(x * rsqrt(mean(x^2) + eps)) with the two roundings of the
// Hugging Face RMSNorm, goes to `xnorm` in global memory, from where every CTA's activation
// producer fetches it with TMA.  The caller closes the phase with a grid barrier.
constexpr int kNormVecs = 4;  // vectors a worker thread holds: rows of up to kNormVecs * kWorkers * 8 = 8192 elements

__device__ __noinline__ void norm_phase(const Ctx& cx, const GemmPhase* ph, int wtid) {
  const KParams& p = *cx.p;
  const int warp = wtid >> 5, lane = wtid & 31;
  // read once: the block barriers below are compiler barriers for memory
  const int m = p.m, k = ph->k, my_cta = cx.cta, grid = cx.grid;
  const float eps = p.eps;
  bf16* const xnorm = p.xnorm;
  const float* const partial = ph->partial;
  const int nvec = k / 8;
  const int parts = ph->add_parts;
  const uint4* wrow = reinterpret_cast<const uint4*>(ph->normw);
  float* red = &cx.misc->sred[0][0];  // kWorkerWarps partial sums (the small-launch kernel's scratch, free here)
  for (int t = my_cta; t < m; t += grid) {
    const uint4* row = reinterpret_cast<const uint4*>(activation_row(p, ph, t));
    uint4 x[kNormVecs];
    float sum = 0.f;
#pragma unroll
    for (int j0 = 0; j0 < kNormVecs; j0 += 2) {
      // two vectors at a time: their residual and partial loads are all issued before any is used
      float4 lo[2][kMaxSplit], hi[2][kMaxSplit];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int v = (j0 + j) * kWorkers + wtid;
        x[j0 + j] = make_uint4(0, 0, 0, 0);
        if (v < nvec) {
          x[j0 + j] = __ldcg(row + v);
#pragma unroll
          for (int s8 = 0; s8 < kMaxSplit; ++s8) {
            if (s8 < parts) {
              const float4* part = reinterpret_cast<const float4*>(partial + (static_cast<size_t>(s8) * m + t) * k) + v * 2;
              lo[j][s8] = __ldcg(part);
              hi[j][s8] = __ldcg(part + 1);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int v = (j0 + j) * kWorkers + wtid;
        if (v >= nvec) continue;
        float f[8];
        unpack8(x[j0 + j], f);
        if (parts > 0) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int s8 = 0; s8 < kMaxSplit; ++s8) {
            if (s8 < parts) {
              acc[0] += lo[j][s8].x; acc[1] += lo[j][s8].y; acc[2] += lo[j][s8].z; acc[3] += lo[j][s8].w;
              acc[4] += hi[j][s8].x; acc[5] += hi[j][s8].y; acc[6] += hi[j][s8].z; acc[7] += hi[j][s8].w;
            }
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = bf16_round(f[e] + bf16_round(acc[e]));
          x[j0 + j] = pack8(f);
        }
        if (ph->h_out) __stcg(reinterpret_cast<uint4*>(ph->h_out + static_cast<size_t>(t) * ph->k) + v, x[j0 + j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum = fmaf(f[e], f[e], sum);
      }
    }
    sum = warp_sum(sum);
    named_bar_sync(1, kWorkers);  // the partial sums of the previous row have been read
    if (lane == 0) red[warp] = sum;
    named_bar_sync(1, kWorkers);
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kWorkerWarps; ++w) total += red[w];
    const float rinv = 1.0f / sqrtf(total / static_cast<float>(k) + eps);
    uint4* out = reinterpret_cast<uint4*>(xnorm + static_cast<size_t>(t) * k);
#pragma unroll
    for (int j = 0; j < kNormVecs; ++j) {
      const int v = j * kWorkers + wtid;
      if (v < nvec) __stcg(out + v, normalise_vec(x[j], __ldg(wrow + v), rinv));
    }
  }
}

// ---------------------------------------------------------------------------
// workers: attention

struct AttnArgs {
  // query of (sequence b, query token qi, head h): q + b*q_bstride + qi*q_ld + h*head_dim
  const bf16* q; long long q_bstride; int q_ld;
  // key/value of (b, position j, kv head g): k + b*kv_bstride + j*kv_ld + g*head_dim
  bf16* k; bf16* v; long long kv_bstride; int kv_ld;
  // decode only: the new token's key/value at knew + b*new_ld + g*head_dim
  const bf16* knew; const bf16* vnew; int new_ld;
  // output of (b, qi, h): out + b*out_bstride + qi*out_tstride + h*out_hstride
  bf16* out; long long out_bstride; int out_tstride; int out_hstride;
  const bf16* mask;   // additive bf16 [batch, 1, sq, klen] or null
  int sq;             // query tokens per sequence (1 in decode)
  int klen;           // keys per sequence (prefill); decode attends len + 1
  int len;            // decode: filled positions before this call (the longest sequence's when lengths are per sequence)
  const int* lens;    // decode with per-sequence valid lengths: filled positions of each sequence; null = `len` for all
  int decode;         // 1: append the new key/value at `len` and attend over [0, len]
  int rope;           // 1: rotate q and the new key while loading (decode)
  int causal;         // prefill without a mask tensor: key j <= query qi
  int combine;        // 1: a split context is summed here into `out`; 0: the consumer sums att_part
  uint32_t stamp;     // value the chunks of this phase publish with their softmax statistics
  float scale;
  const CUtensorMap *kmap, *vmap;  // decode: tiled descriptors of the two caches (see attention_decode), or null
};

__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, int style, float& first, float& second) {
  if (style == MK_ROPE_HALF_SWAP) {
    const float a = bf16_round(x1 * c), b = bf16_round(x2 * s);
    first = bf16_round(a - b);
    second = bf16_round(b + a);
  } else {
    first = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * s));
    second = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
  }
}

// How many chunks the context of a decode attention phase is cut into.
__device__ __forceinline__ int decode_chunks(int keys, int rows, int grid, int gs, int score_bytes = kScoreBytes) {
  const int max_len = (score_bytes / 4 / gs) & ~7;
  int nch = grid / rows;
  if (nch < 1) nch = 1;
  const int by_len = (keys + 63) / 64;
  if (nch > by_len) nch = by_len;
  if (nch > kMaxChunks) nch = kMaxChunks;
  const int need = (keys + max_len - 1) / max_len;
  if (nch < need) nch = need;
  return nch;
}

// Decode attention (one query token per sequence) as a stream of cache tiles.
// A unit is one (sequence, group of adjacent KV heads, context chunk).  The cache is
// [batch, capacity, kv_heads, head_dim]: one KV head's rows are 128-256 byte pieces a whole cache
// row apart, which DRAM serves at a fraction of its rate, so a unit takes as many adjacent KV heads
// as its query heads allow (up to eight query heads per unit): every cached position then
// contributes one contiguous run of up to 1 KB.  The K rows and then the V rows of the unit travel
// through three shared-memory stages with cp.async (each head's rows in a sub-tile of its own, so
// the inner loops see the same [key][128 or 256 B] tile as for a single head): while the workers
// take the scores (or the value sums) of one tile, the next two tiles are in flight.  The new
// position's key/value rows are not in the cache yet: they are patched into their tile from shared
// memory.  Arithmetic and rounding points are those described above attention_phase for decode;
// the exchange of the chunk statistics and the hand-over of the chunk partials are the same
// protocol as there.
// The stages live in the weight ring, which is idle during attention (the weight producer waits at the
// projection that follows, GemmPhase::gate): three stages of 32 KB keep two tiles, 64 KB per SM, in
// flight.
static_assert(kScoreBytes + kDecScratchBytes <= kBBytes, "scores and scratch exceed their region");
static_assert(kDecStages * kDecTileBytes <= kRingBytes, "cache stages exceed the weight ring");

// KV heads one decode-attention unit covers: the largest divisor of kv_heads that keeps the unit at
// eight query heads and 1 KB of cache row (512 elements) or fewer.
__host__ __device__ inline int decode_heads_per_unit(int kv_heads, int gs, int head_dim) {
  int hpu = 8 / gs;
  if (hpu > 512 / head_dim) hpu = 512 / head_dim;
  if (hpu < 1) hpu = 1;
  while (kv_heads % hpu) --hpu;
  return hpu;
}

// Copy `count` cached positions of `hpu` adjacent heads (head_dim bf16 each, contiguous in a cache row;
// rows `ld` elements apart) into a stage, except position `skip`.  Head h's rows form a sub-tile of
// `tile_keys` rows at dst + h * tile_keys * row_bytes; piece p of row r lands at piece p ^ (r & 7) of
// its 128-byte group, so that a column of pieces spreads over all banks.
__device__ __noinline__ void fetch_cache_tile(uint32_t dst, const bf16* src, int ld, int count, int skip, int hd, int hpu,
                                              int tile_keys, int wtid) {
  const int shift = (hd == 64) ? 3 : 4;          // 16-byte pieces per head row: 8 or 16
  const int per_key = hpu << shift;              // pieces per cached position: a power of two times hpu, at most 64
  const uint32_t row_bytes = static_cast<uint32_t>(hd) * 2u;
  // A thread keeps its (head, piece) column and walks down the positions in steps of kWorkers / per_key,
  // so that both addresses advance by constants (per_key divides kWorkers for every supported shape but
  // hpu in {3, 5, 6, 7}, which take the general loop).
  if (kWorkers % per_key == 0) {
    int rest, step, key;
    if ((per_key & (per_key - 1)) == 0) {  // a power of two (1, 2, 4 or 8 heads): shifts, no division
      const int sh = 31 - __clz(per_key);
      rest = wtid & (per_key - 1);
      step = kWorkers >> sh;
      key = wtid >> sh;
    } else {
      rest = wtid % per_key;
      step = kWorkers / per_key;
      key = wtid / per_key;
    }
    const int head = rest >> shift, piece = rest & ((1 << shift) - 1);
    const uint4* from = reinterpret_cast<const uint4*>(src + static_cast<long long>(key) * ld) + rest;
    const long long from_step = static_cast<long long>(step) * ld / 8;  // in 16-byte units: ld is a multiple of 8
    uint32_t to = dst + (static_cast<uint32_t>(head) * tile_keys + key) * row_bytes;
    const uint32_t to_step = step * row_bytes;
#pragma unroll 4
    for (; key < count; key += step) {
      if (key != skip) cp_async16(to + ((piece ^ (key & 7)) << 4), from);
      to += to_step;
      from += from_step;
    }
    return;
  }
  const int total = count * per_key;
#pragma unroll 2
  for (int it = wtid; it < total; it += kWorkers) {
    const int key = it / per_key, rest = it - key * per_key;
    const int head = rest >> shift, piece = rest & ((1 << shift) - 1);
    if (key != skip)
      cp_async16(dst + (static_cast<uint32_t>(head) * tile_keys + key) * row_bytes + ((piece ^ (key & 7)) << 4),
                 reinterpret_cast<const uint4*>(src + static_cast<long long>(key) * ld) + rest);
  }
}

__device__ __noinline__ bool attention_decode(const Ctx& cx, const AttnArgs& A_in, int wtid) {
  // Private copies of the arguments and of the parameters this phase reads: every poll, copy wait and block
  // barrier below is a compiler barrier for memory, behind which a value that lives behind a reference is
  // loaded again (a kernel parameter through the context: two dependent loads).
  const AttnArgs A = A_in;
  struct {
    int head_dim, q_heads, kv_heads, batch, max_positions, rope_style, prefill_rope_style, m;
    const bf16 *cos_t, *sin_t;
    float *att_xch, *att_part;
    long long* pos;
  } p = {cx.p->head_dim, cx.p->q_heads, cx.p->kv_heads, cx.p->batch, cx.p->max_positions, cx.p->rope_style,
         cx.p->prefill_rope_style, cx.p->m, cx.p->cos_t, cx.p->sin_t, cx.p->att_xch, cx.p->att_part, cx.p->pos};
  const int hd = p.head_dim, half = hd / 2;
  const int gs = p.q_heads / p.kv_heads;
  const int hpu = decode_heads_per_unit(p.kv_heads, gs, hd);  // KV heads per unit
  const int G = gs * hpu;                                  // query heads per unit (<= 8)
  const int groups = p.kv_heads / hpu;
  const int rows = p.batch * groups;
  const int n_max = A.len + 1;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int lpk = hd / 8;  // 16-byte pieces per head row
  const int nch = decode_chunks(n_max, rows, cx.grid, G);
  const int chunk = (n_max + nch - 1) / nch;
  const int units = rows * nch;
  const int row_bytes = hd * 2;
  const int tile_keys = kDecTileBytes / (row_bytes * hpu);
  const int sub_bytes = tile_keys * row_bytes;     // one head's sub-tile
  const int stage_bytes = sub_bytes * hpu;

  float* sc = reinterpret_cast<float*>(cx.smem_b);                                      // [G][chunk]
  uint8_t* tiles = cx.smem_a;                                                           // [stages][hpu][tile_keys][hd] bf16, in the weight ring
  float* qs = reinterpret_cast<float*>(cx.smem_b + kBBytes - kDecScratchBytes);         // [G][hd]
  float* red = qs + 8 * 128;                                                            // [worker warps][8] x 2, then [parts][G*hd]
  bf16* kn = reinterpret_cast<bf16*>(red + 1024);                                       // [hpu][hd]
  bf16* vn = kn + 512;                                                                  // [hpu][hd]
  float* stat = reinterpret_cast<float*>(vn + 512);                                     // [16]: max[8], sum[8]
  const uint32_t tiles_addr = smem_u32(tiles);

  // value accumulation: an item is (part of the keys, query head of the unit, 16-byte piece of the output row);
  // part q takes keys q, q + parts, ... of every tile; the fp32 sums of an item stay in `red` between tiles
  const int cols = G * hd;
  const int pieces = G * lpk;
  int parts = kWorkers / pieces;
  if (parts * cols > 1024) parts = 1024 / cols;
  if (parts < 1) parts = 1;
  const int items = parts * pieces;  // <= kWorkers
  const int item_part = wtid / pieces, item_g = (wtid - item_part * pieces) / lpk, item_piece = wtid % lpk;

#pragma unroll 1
  for (int u = cx.cta; u < units; u += cx.grid) {
    const int rowg = u / nch, ch = u - rowg * nch;
    const int b = rowg / groups, kvh0 = (rowg - b * groups) * hpu;  // first KV head of the unit
    const int filled = A.lens ? A.lens[b] : A.len;  // this sequence's cached positions; chunks past its end are empty
    const int j0 = ch * chunk;
    const int j1 = min(filled + 1, j0 + chunk);
    const int cl = max(0, j1 - j0);
    const int newpos = filled;
    const bool owner = (filled >= j0 && filled < j1);
    const int nt = (cl + tile_keys - 1) / tile_keys;
    const bf16* kbase = A.k + b * A.kv_bstride + kvh0 * hd;
    const bf16* vbase = A.v + b * A.kv_bstride + kvh0 * hd;
    named_bar_sync(1, kWorkers);  // previous unit is done with the scratch and the stages

    // Element s of the stream is K tile s (s < nt) or V tile s - nt; it uses stage s % kDecStages.
    // Every call commits one group, an empty one past the end, so that the group count is uniform.
    auto issue = [&](int s) {
      if (s < 2 * nt) {
        const int t = (s < nt) ? s : s - nt;
        const int t0 = j0 + t * tile_keys, t1 = min(j1, t0 + tile_keys);
        fetch_cache_tile(tiles_addr + (s % kDecStages) * stage_bytes,
                         ((s < nt) ? kbase : vbase) + static_cast<long long>(t0) * A.kv_ld, A.kv_ld, t1 - t0, newpos - t0,
                         hd, hpu, tile_keys, wtid);
      }
      cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kDecStages - 1; ++s) issue(s);

    // --- q of every query head of the unit and the new keys (rotated if asked), and the new values
    {
      long long pos = 0;
      if (A.rope) {
        pos = p.pos[b];
        if (pos < 0 || pos >= p.max_positions) pos = 0;  // reported by the prologue
      }
#pragma unroll 1
      for (int idx = wtid; idx < (G + hpu) * half; idx += kWorkers) {
        const int g = idx / half, i = idx - g * half;  // g < G: query head g of the unit; else new key of KV head g - G
        const bf16* src = (g < G) ? A.q + b * A.q_bstride + (kvh0 * gs + g) * hd
                                  : A.knew + static_cast<long long>(b) * A.new_ld + (kvh0 + g - G) * hd;
        float first = ldcg_bf16(src + i);
        float second = ldcg_bf16(src + i + half);
        if (A.rope) {
          const float c = ldg_bf16(p.cos_t + pos * hd + i);
          const float sn = ldg_bf16(p.sin_t + pos * hd + i);
          rope_pair(first, second, c, sn, p.rope_style, first, second);
        }
        if (g < G) {
          qs[g * hd + i] = first;
          qs[g * hd + i + half] = second;
        } else {
          kn[(g - G) * hd + i] = __float2bfloat16_rn(first);
          kn[(g - G) * hd + i + half] = __float2bfloat16_rn(second);
        }
      }
#pragma unroll 1
      for (int i = wtid; i < hpu * hd; i += kWorkers)
        vn[i] = __float2bfloat16_rn(ldcg_bf16(A.vnew + static_cast<long long>(b) * A.new_ld + kvh0 * hd + i));
    }
    named_bar_sync(1, kWorkers);
    if (owner) {  // in-kernel KV append: the unit's heads are adjacent in the cache row
      bf16* kd = A.k + b * A.kv_bstride + static_cast<long long>(filled) * A.kv_ld + kvh0 * hd;
      bf16* vd = A.v + b * A.kv_bstride + static_cast<long long>(filled) * A.kv_ld + kvh0 * hd;
#pragma unroll 1
      for (int i = wtid; i < hpu * hd; i += kWorkers) {
        kd[i] = kn[i];
        vd[i] = vn[i];
      }
    }
    // The new position's row joins its tile (its row was not fetched): one 16-byte piece per thread.
    auto patch = [&](uint8_t* tile, const bf16* fresh, int local) {
      if (wtid < hpu * lpk) {
        const int head = wtid / lpk, piece = wtid - head * lpk;
        *reinterpret_cast<uint4*>(tile + head * sub_bytes + local * row_bytes + ((piece ^ (local & 7)) << 4)) =
            *reinterpret_cast<const uint4*>(fresh + head * hd + piece * 8);
      }
    };

    // --- scores: one thread per (query head of the unit, key), a head_dim-term fp32 chain each
#pragma unroll 1
    for (int s = 0; s < nt; ++s) {
      const int t0 = j0 + s * tile_keys, t1 = min(j1, t0 + tile_keys);
      uint8_t* tile = tiles + (s % kDecStages) * stage_bytes;
      cp_async_wait_group<kDecStages - 2>();  // this thread's pieces of tile s have landed
      if (newpos >= t0 && newpos < t1) patch(tile, kn, newpos - t0);
      named_bar_sync(1, kWorkers);  // tile s is complete; every thread is done with tile s - 1
      issue(s + kDecStages - 1);
      const int tk = t1 - t0;
      const int tk_shift = (tk & (tk - 1)) == 0 ? 31 - __clz(tk) : -1;  // full tiles hold a power of two of keys
#pragma unroll 1
      for (int item = wtid; item < G * tk; item += kWorkers) {
        const int g = tk_shift >= 0 ? item >> tk_shift : item / tk, key = item - g * tk;
        const uint8_t* krow = tile + (g / gs) * sub_bytes + key * row_bytes;
        const float* qv = qs + g * hd;
        // four partial sums (pieces 0, 4, 8, ... / 1, 5, ... / ...): the chains have to be independent
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int piece0 = 0; piece0 < lpk; piece0 += 4) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int piece = piece0 + c;
            float kf[8];
            unpack8(*reinterpret_cast<const uint4*>(krow + ((piece ^ (key & 7)) << 4)), kf);
            const float4 qa = *reinterpret_cast<const float4*>(qv + piece * 8);
            const float4 qb = *reinterpret_cast<const float4*>(qv + piece * 8 + 4);
            float acc = part[c];
            acc = fmaf(qa.x, kf[0], acc); acc = fmaf(qa.y, kf[1], acc); acc = fmaf(qa.z, kf[2], acc); acc = fmaf(qa.w, kf[3], acc);
            acc = fmaf(qb.x, kf[4], acc); acc = fmaf(qb.y, kf[5], acc); acc = fmaf(qb.z, kf[6], acc); acc = fmaf(qb.w, kf[7], acc);
            part[c] = acc;
          }
        }
        const float dot = (part[0] + part[1]) + (part[2] + part[3]);
        sc[g * chunk + (t0 - j0) + key] = bf16_round(dot) * A.scale;
      }
    }
    named_bar_sync(1, kWorkers);

    // --- chunk max, then chunk sum of exp(score - chunk max); the first V tiles are in flight meanwhile
#pragma unroll 1
    for (int g = 0; g < G; ++g) {
      float m = -INFINITY;
#pragma unroll 1
      for (int i = wtid; i < cl; i += kWorkers) m = fmaxf(m, sc[g * chunk + i]);
      m = warp_max(m);
      if (lane == 0) red[warp * 8 + g] = m;
    }
    named_bar_sync(1, kWorkers);
#pragma unroll 1
    for (int g = 0; g < G; ++g) {
      float m = red[g];
#pragma unroll
      for (int w = 1; w < kWorkerWarps; ++w) m = fmaxf(m, red[w * 8 + g]);
      float sum = 0.f;
#pragma unroll 1
      for (int i = wtid; i < cl; i += kWorkers) sum += expf(sc[g * chunk + i] - m);
      sum = warp_sum(sum);
      if (lane == 0) red[kWorkerWarps * 8 + warp * 8 + g] = sum;
      if (wtid == 0) stat[g] = m;
    }
    named_bar_sync(1, kWorkers);
    if (wtid < G) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kWorkerWarps; ++w) total += red[kWorkerWarps * 8 + w * 8 + wtid];
      stat[8 + wtid] = total;
    }
    named_bar_sync(1, kWorkers);

    if (nch > 1) {
      // --- publish (max, sum) with this phase's stamp; wait for every chunk of the row group
      float* mine = p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + ch) * kExchangeFloats;
      if (wtid < 16) __stcg(mine + wtid, stat[wtid]);
      __threadfence();
      named_bar_sync(1, kWorkers);
      if (wtid == 0) st_relaxed_u32(reinterpret_cast<uint32_t*>(mine + kXchStatsFlag), A.stamp);
      bool ok = true;
      if (wtid < nch) {
        const uint32_t* theirs = reinterpret_cast<const uint32_t*>(
            p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + wtid) * kExchangeFloats + kXchStatsFlag);
        uint32_t spins = 0;
        while (ld_relaxed_u32(theirs) != A.stamp) {
          if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, rowg)) {
            ok = false;
            break;
          }
        }
        __threadfence();
      }
      if (!workers_ok(cx, ok)) {
        cp_async_wait_all();  // nothing of this CTA stays in flight past the return
        return false;
      }
      if (wtid < G) {
        const float* all = p.att_xch + static_cast<size_t>(rowg) * kMaxChunks * kExchangeFloats;
        float m = -INFINITY;
        for (int c = 0; c < nch; ++c) m = fmaxf(m, __ldcg(all + c * kExchangeFloats + wtid));
        float sum = 0.f;
        for (int c = 0; c < nch; ++c)
          sum += __ldcg(all + c * kExchangeFloats + 8 + wtid) * expf(__ldcg(all + c * kExchangeFloats + wtid) - m);
        stat[wtid] = m;
        stat[8 + wtid] = sum;
      }
      named_bar_sync(1, kWorkers);
    }

    // --- probabilities (bf16, against the global max and sum)
#pragma unroll 1
    for (int g = 0; g < G; ++g) {
      const float m = stat[g], denom = stat[8 + g];
#pragma unroll 1
      for (int i = wtid; i < cl; i += kWorkers) sc[g * chunk + i] = bf16_round(expf(sc[g * chunk + i] - m) / denom);
    }
    // --- value sums, tile by tile
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int s = nt; s < 2 * nt; ++s) {
      const int t0 = j0 + (s - nt) * tile_keys, t1 = min(j1, t0 + tile_keys);
      uint8_t* tile = tiles + (s % kDecStages) * stage_bytes;
      cp_async_wait_group<kDecStages - 2>();
      if (newpos >= t0 && newpos < t1) patch(tile, vn, newpos - t0);  // the new value rows join their tile
      named_bar_sync(1, kWorkers);  // the tile is complete and (first tile) so are the probabilities
      issue(s + kDecStages - 1);
      const int tk = t1 - t0;
      if (wtid < items) {  // at most one item per thread: its sums stay in registers across the tiles
        const float* pr = sc + item_g * chunk + (t0 - j0);
        const uint8_t* vtile = tile + (item_g / gs) * sub_bytes;
#pragma unroll 4
        for (int kk = item_part; kk < tk; kk += parts) {
          float vf[8];
          unpack8(*reinterpret_cast<const uint4*>(vtile + kk * row_bytes + ((item_piece ^ (kk & 7)) << 4)), vf);
          const float w = pr[kk];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, vf[e], acc[e]);
        }
      }
    }
    if (wtid < items) {
      float* mine = red + (item_part * G + item_g) * hd + item_piece * 8;
      *reinterpret_cast<float4*>(mine) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(mine + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    named_bar_sync(1, kWorkers);
#pragma unroll 1
    for (int col = wtid; col < cols; col += kWorkers) {
      float o = red[col];
#pragma unroll 1
      for (int part = 1; part < parts; ++part) o += red[part * cols + col];
      const int g = col / hd, d = col - g * hd;
      const int head = kvh0 * gs + g;
      if (nch == 1) {
        A.out[b * A.out_bstride + head * A.out_hstride + d] = __float2bfloat16_rn(o);
      } else {
        const size_t row = static_cast<size_t>(b) * p.q_heads + head;
        __stcg(p.att_part + (row * kMaxChunks + ch) * hd + d, o);
      }
    }
    if (nch > 1 && A.combine) {
      // There is no consumer phase that adds chunk partials: chunk 0's CTA waits for the partials of its
      // peers (second stamp) and sums them in chunk order.
      float* mine = p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + ch) * kExchangeFloats;
      __threadfence();
      named_bar_sync(1, kWorkers);
      if (wtid == 0) st_relaxed_u32(reinterpret_cast<uint32_t*>(mine + kXchPartsFlag), A.stamp);
      if (ch == 0) {
        bool ok = true;
        if (wtid < nch) {
          const uint32_t* theirs = reinterpret_cast<const uint32_t*>(
              p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + wtid) * kExchangeFloats + kXchPartsFlag);
          uint32_t spins = 0;
          while (ld_relaxed_u32(theirs) != A.stamp) {
            if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, rowg)) {
              ok = false;
              break;
            }
          }
          __threadfence();
        }
        if (!workers_ok(cx, ok)) {
          cp_async_wait_all();
          return false;
        }
        for (int idx = wtid; idx < cols; idx += kWorkers) {
          const int g = idx / hd, d = idx - g * hd;
          const int head = kvh0 * gs + g;
          const size_t row = static_cast<size_t>(b) * p.q_heads + head;
          float o = 0.f;
          for (int c = 0; c < nch; ++c) o += __ldcg(p.att_part + (row * kMaxChunks + c) * hd + d);
          A.out[b * A.out_bstride + head * A.out_hstride + d] = __float2bfloat16_rn(o);
        }
      }
    }
  }
  return true;
}

// The same phase as a stream without a block barrier per tile, for long chunks and caches the host has
// described (AttnArgs::kmap / vmap): one tiled TMA copy brings a stage (64 dimensions x tile_keys positions x
// the unit's 64-dimension chunks, 128-byte swizzled: [chunk][key][128 B]), both products run on mma.sync
// (scores: D[16 keys][heads] = K tile x q; values: D[16 dims][heads] += V tile^T x p), warp w works for KV
// head w % hpu, waits for a stage's `full` barrier and releases it on its `empty` barrier; the copies are
// issued by the weight producer (serve_cache_stream), which refills a stage the moment its eight releases
// are in.  The block meets only around what is exchanged between warps: the scores -> statistics ->
// probabilities hand-over and the tiles that are written by hand (new row, zeroed tail).  Measured on the
// 1.7B shape at context 1024, per step against attention_decode: batch 8 / 16 / 32 (chunks of 256 / 513 /
// 1025 keys) 16 % / 18 % / 21 % faster; chunks shorter than four tiles never fill the pipeline and stay
// with attention_decode, hence decode_stream_ok().
__device__ __forceinline__ bool decode_stream_ok(const KParams& p, const AttnArgs& A, int grid) {
  if (A.kmap == nullptr) return false;
  const int gs = p.q_heads / p.kv_heads, hd = p.head_dim;
  const int hpu = decode_heads_per_unit(p.kv_heads, gs, hd);
  const int tile_keys = kDecTileBytes / (hd * 2 * hpu);
  if ((hpu & (hpu - 1)) != 0 || (tile_keys & 15) != 0) return false;
  const int n_max = A.len + 1;
  const int nch = decode_chunks(n_max, p.batch * (p.kv_heads / hpu), grid, gs * hpu);
  return (n_max + nch - 1) / nch >= 4 * tile_keys;
}

__device__ __noinline__ bool attention_decode_stream(const Ctx& cx, const AttnArgs& A_in, int wtid) {
  // Private copies of the arguments and of the parameters this phase reads: every poll, copy wait and block
  // barrier below is a compiler barrier for memory, behind which a value that lives behind a reference is
  // loaded again (a kernel parameter through the context: two dependent loads).
  const AttnArgs A = A_in;
  struct {
    int head_dim, q_heads, kv_heads, batch, max_positions, rope_style;
    const bf16 *cos_t, *sin_t;
    float *att_xch, *att_part;
    long long* pos;
  } p = {cx.p->head_dim, cx.p->q_heads, cx.p->kv_heads, cx.p->batch, cx.p->max_positions, cx.p->rope_style,
         cx.p->cos_t,    cx.p->sin_t,   cx.p->att_xch,  cx.p->att_part, cx.p->pos};
  const int hd = p.head_dim, half = hd / 2;
  const int gs = p.q_heads / p.kv_heads;
  const int hpu = decode_heads_per_unit(p.kv_heads, gs, hd);  // KV heads per unit
  const int G = gs * hpu;                                  // query heads per unit (<= 8)
  const int groups = p.kv_heads / hpu;
  const int rows = p.batch * groups;
  const int n_max = A.len + 1;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int lpk = hd / 8;  // 16-byte pieces per head row
  const int nch = decode_chunks(n_max, rows, cx.grid, G);
  const int chunk = (n_max + nch - 1) / nch;
  const int units = rows * nch;
  const int row_bytes = hd * 2;
  const int tile_keys = kDecTileBytes / (row_bytes * hpu);
  const int stage_bytes = tile_keys * row_bytes * hpu;

  float* sc = reinterpret_cast<float*>(cx.smem_b);                                      // [G][chunk]
  uint8_t* tiles = cx.smem_a;                                                           // [stages][hpu][tile_keys][hd] bf16, in the weight ring
  float* red = reinterpret_cast<float*>(cx.smem_b + kBBytes - kDecScratchBytes) + 8 * 128;  // [G * hd] value sums (same carve-up as attention_decode)
  bf16* kn = reinterpret_cast<bf16*>(red + 1024);                                       // [hpu][hd]
  bf16* vn = kn + 512;                                                                  // [hpu][hd]
  float* stat = reinterpret_cast<float*>(vn + 512);                                     // [16]: max[8], sum[8]
  bf16* qb = reinterpret_cast<bf16*>(stat + 16);                                        // [G][hd], q again as bf16 (exact)
  const uint32_t tiles_addr = smem_u32(tiles);
  // Both products run on the warp-level tensor cores (the caller checked with decode_stream_ok() that the
  // unit's KV heads divide the eight worker warps): one mma.sync (m16n8k16) multiplies 16 cached positions x
  // 16 head dimensions by the (up to eight) query heads of a KV head, where the CUDA-core loops of
  // attention_decode need 17 instructions per lane for eight elements and keep that phase, not the cache
  // stream, bound by instruction issue.
  //   scores:  D[16 keys][heads]  = K tile (ldmatrix)        x q[dims][heads]   (q fragments stay in registers)
  //   values:  D[16 dims][heads] += V tile^T (ldmatrix.trans) x p[keys][heads]
  // Warp w works for KV head w % hpu; the 8 / hpu warps of a head split the 16-key blocks (scores) and
  // the 16-dimension tiles of the output row (values).
  // Tensor-core layout of a stage: the unit's cache rows as sub-tiles of 64 dimensions, [chunk][key][128 B]
  // with the 16-byte pieces of a row exchanged by key % 8 (the 128-byte swizzle of a tiled TMA copy),
  // chunk = head * (head_dim / 64) + dimension / 64.
  const int cph = hd / 64;                       // chunks per head
  const uint32_t csub = tile_keys * 128u;        // one chunk's sub-tile
  auto piece_at = [&](uint32_t stage, int head, int key, int piece) -> uint32_t {
    return stage + (head * cph + (piece >> 3)) * csub + key * 128u + (((piece & 7) ^ (key & 7)) << 4);
  };
  // One tiled TMA copy brings a whole stage (box = 64 dimensions x tile_keys positions x the unit's chunks);
  // cp.async, 16 bytes per thread and request, measured 17 GB/s per SM on this stream, a third of an SM's share
  // of HBM.
  const uint32_t kvfull0 = smem_u32(&cx.tc->kvfull[0]), kvempty0 = smem_u32(&cx.tc->kvempty[0]);
  int gtile = cx.tc->kv_seq;  // cache tiles issued by this CTA before this unit (same value in every thread)
  const int my_head = warp & (hpu - 1), head_warps = kWorkerWarps / hpu, my_slot = warp / hpu;
  const int ksteps = hd / 16, dim_tiles = hd / 16;
  const int lg = lane >> 2, lt = lane & 3;
  const int cols = G * hd;

#pragma unroll 1
  for (int u = cx.cta; u < units; u += cx.grid) {
    const int rowg = u / nch, ch = u - rowg * nch;
    const int b = rowg / groups, kvh0 = (rowg - b * groups) * hpu;  // first KV head of the unit
    const int filled = A.lens ? A.lens[b] : A.len;  // this sequence's cached positions; chunks past its end are empty
    const int j0 = ch * chunk;
    const int j1 = min(filled + 1, j0 + chunk);
    const int cl = max(0, j1 - j0);
    const int newpos = filled;
    const bool owner = (filled >= j0 && filled < j1);
    const int nt = (cl + tile_keys - 1) / tile_keys;
    named_bar_sync(1, kWorkers);  // previous unit is done with the scratch and the stages

    // Element s of the stream is K tile s (s < nt) or V tile s - nt; it uses stage (gtile + s) % kDecStages.
    // The copies are the weight producer's: it waits at the projection that follows this phase, takes the
    // request below and issues a stage's next copy as soon as every worker warp has released the stage, so
    // all the stages but the one being read stay in flight and no worker spends time on issuing.
    auto stage_of = [&](int s) -> int { return (gtile + s) % kDecStages; };
    if (wtid == 0) {
      SmemMiscTc* tc = cx.tc;
      tc->kvr.kmap = A.kmap;
      tc->kvr.vmap = A.vmap;
      tc->kvr.t0 = j0;
      tc->kvr.nt = nt;
      tc->kvr.tile_keys = tile_keys;
      tc->kvr.chunk0 = kvh0 * cph;
      tc->kvr.b = b;
      tc->kvr.gtile = gtile;
      tc->kvr.stage_bytes = static_cast<uint32_t>(stage_bytes);
      __threadfence_block();
      *reinterpret_cast<volatile int*>(&tc->kv_req) = tc->kv_req + 1;
    }
    // Tile s of the unit has landed (every thread waits: a copy's bytes are visible to the threads that saw its barrier flip).
    auto landed = [&](int s) -> bool {
      return wait_mbar(cx, kvfull0 + stage_of(s) * 8u, ((gtile + s) / kDecStages) & 1, SITE_KV_TILE, s);
    };

    // --- q of every query head of the unit and the new keys (rotated if asked), and the new values: one thread
    // per pair of 16-byte vectors (elements i..i+7 and i+half..), every load of the phase in one round trip
    {
      long long pos = 0;
      if (A.rope) {
        pos = p.pos[b];
        if (pos < 0 || pos >= p.max_positions) pos = 0;  // reported by the prologue
      }
      const int vecs = half / 8;
      const int rot_items = (G + hpu) * vecs;  // <= 128
      const int v_items = hpu * hd / 8;        // <= 64
      if (wtid < rot_items) {
        const int g = wtid / vecs, i = (wtid - g * vecs) * 8;  // g < G: query head g of the unit; else new key of KV head g - G
        const bf16* src = (g < G) ? A.q + b * A.q_bstride + (kvh0 * gs + g) * hd
                                  : A.knew + static_cast<long long>(b) * A.new_ld + (kvh0 + g - G) * hd;
        float first[8], second[8];
        unpack8(__ldcg(reinterpret_cast<const uint4*>(src + i)), first);
        unpack8(__ldcg(reinterpret_cast<const uint4*>(src + i + half)), second);
        if (A.rope) {
          float c[8], sn[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.cos_t + pos * hd + i)), c);
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.sin_t + pos * hd + i)), sn);
#pragma unroll
          for (int e = 0; e < 8; ++e) rope_pair(first[e], second[e], c[e], sn[e], p.rope_style, first[e], second[e]);
        }
        bf16* dst = (g < G) ? qb + g * hd : kn + (g - G) * hd;  // exact: the rotated values are bf16 values
        *reinterpret_cast<uint4*>(dst + i) = pack8(first);
        *reinterpret_cast<uint4*>(dst + i + half) = pack8(second);
      } else if (wtid >= 128 && wtid - 128 < v_items) {
        const int i = (wtid - 128) * 8;
        *reinterpret_cast<uint4*>(vn + i) =
            __ldcg(reinterpret_cast<const uint4*>(A.vnew + static_cast<long long>(b) * A.new_ld + kvh0 * hd + i));
      }
    }
    named_bar_sync(1, kWorkers);
    trace_event(cx, wtid, EV_ATT_INPUTS);
    uint32_t qfrag[8][2];  // B fragments of this warp's KV head: q[dims][query heads], one pair per 16 dimensions
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qfrag[ks][0] = qfrag[ks][1] = 0u;
      if (ks < ksteps && lg < gs) {
        const bf16* at = qb + (my_head * gs + lg) * hd + ks * 16 + lt * 2;
        qfrag[ks][0] = *reinterpret_cast<const uint32_t*>(at);
        qfrag[ks][1] = *reinterpret_cast<const uint32_t*>(at + 8);
      }
    }
    if (owner) {  // in-kernel KV append: the unit's heads are adjacent in the cache row
      bf16* kd = A.k + b * A.kv_bstride + static_cast<long long>(filled) * A.kv_ld + kvh0 * hd;
      bf16* vd = A.v + b * A.kv_bstride + static_cast<long long>(filled) * A.kv_ld + kvh0 * hd;
#pragma unroll 1
      for (int i = wtid; i < hpu * hd; i += kWorkers) {
        kd[i] = kn[i];
        vd[i] = vn[i];
      }
    }
    // The new position's row joins its tile (its row was not fetched): one 16-byte piece per thread.
    auto patch = [&](uint8_t* tile, const bf16* fresh, int local) {
      if (wtid < hpu * lpk) {
        const int head = wtid / lpk, piece = wtid - head * lpk;
        uint8_t* at = tile + piece_at(0u, head, local, piece);
        *reinterpret_cast<uint4*>(at) = *reinterpret_cast<const uint4*>(fresh + head * hd + piece * 8);
      }
    };
    bool tiles_ok = true;

    // A tile is done with (this warp's share): one arrival per warp frees its stage for the copy S - 1 tiles on.
    auto release = [&](int s) {
      __syncwarp();
      if (lane == 0) mbar_arrive(kvempty0 + stage_of(s) * 8u);
    };
    // --- scores, pipelined: no block barrier per tile.  A warp waits for the tile's copy, takes the scores of
    // its head's key blocks and releases the stage; the weight producer refills it.
    // Only the tile that holds the new position needs the block (its row is patched in by a few threads).
#pragma unroll 1
    for (int s = 0; s < nt; ++s) {
      const int t0 = j0 + s * tile_keys, t1 = min(j1, t0 + tile_keys);
      uint8_t* tile = tiles + stage_of(s) * stage_bytes;
      tiles_ok = landed(s) && tiles_ok;
      if (newpos >= t0 && newpos < t1) {
        patch(tile, kn, newpos - t0);
        fence_proxy_async_all();
        named_bar_sync(1, kWorkers);
      }
      const int tk = t1 - t0;
      const uint32_t stage = smem_u32(tile);
#pragma unroll 1
      for (int blk = my_slot; blk * 16 < tk; blk += head_warps) {
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        const int row = blk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll 2
        for (int ks = 0; ks < ksteps; ++ks) {
          uint32_t af[4];
          ldmatrix_x4(af, piece_at(stage, my_head, row, ks * 2 + (lane >> 4)));
          mma_bf16_16816(d, af, qfrag[ks][0], qfrag[ks][1]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = blk * 16 + lg + (e >> 1) * 8, n = lt * 2 + (e & 1);
          if (n < gs && key < tk) sc[(my_head * gs + n) * chunk + (t0 - j0) + key] = bf16_round(d[e]) * A.scale;
        }
      }
      release(s);
    }
    named_bar_sync(1, kWorkers);
    trace_event(cx, wtid, EV_ATT_SCORES);

    // --- chunk max and chunk sum of exp(score - chunk max); the first V tiles are in flight meanwhile.  Warp g
    // owns query head g of the unit (at most eight): no block barrier until every head's numbers are in `stat`.
    {
      bool fresh = true;
      if (warp < G) {
        const float* mine = sc + warp * chunk;
        float m = -INFINITY;
#pragma unroll 1
        for (int i = lane; i < cl; i += 32) m = fmaxf(m, mine[i]);
        m = warp_max(m);
        float sum = 0.f;
#pragma unroll 1
        for (int i = lane; i < cl; i += 32) sum += expf(mine[i] - m);
        sum = warp_sum(sum);
        if (nch > 1) {
          // publish (max, sum), each with this phase's stamp in one 64-bit word (a reader that sees the stamp has
          // the value: no fence, no flag), and wait for the same two words of every chunk of the row group
          constexpr int kWords = kExchangeFloats / 2;
          unsigned long long* rec = reinterpret_cast<unsigned long long*>(p.att_xch) +
                                    static_cast<size_t>(rowg) * kMaxChunks * kWords;
          const unsigned long long tag = static_cast<unsigned long long>(A.stamp) << 32;
          if (lane == 0) {
            st_relaxed_u64(rec + ch * kWords + warp, tag | __float_as_uint(m));
            st_relaxed_u64(rec + ch * kWords + 8 + warp, tag | __float_as_uint(sum));
          }
          float cm = -INFINITY, cs = 0.f;
          if (lane < nch) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
              const unsigned long long* word = rec + lane * kWords + which * 8 + warp;
              unsigned long long w = ld_relaxed_u64(word);
              uint32_t spins = 0;
              while (static_cast<uint32_t>(w >> 32) != A.stamp) {
                if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, rowg)) {
                  fresh = false;
                  break;
                }
                w = ld_relaxed_u64(word);
              }
              const float value = __uint_as_float(static_cast<uint32_t>(w));
              if (which == 0) cm = value; else cs = value;
            }
          }
          m = warp_max(cm);
          sum = 0.f;  // in chunk order, as one thread would add them
#pragma unroll 1
          for (int c = 0; c < nch; ++c)
            sum += __shfl_sync(0xffffffffu, cs, c) * expf(__shfl_sync(0xffffffffu, cm, c) - m);
        }
        if (lane == 0) {
          stat[warp] = m;
          stat[8 + warp] = sum;
        }
      }
      if (!workers_ok(cx, fresh)) {
        cp_async_wait_all();  // nothing of this CTA stays in flight past the return
        return false;
      }
    }

    trace_event(cx, wtid, EV_ATT_STATS);
    // --- probabilities (bf16, against the global max and sum)
#pragma unroll 1
    for (int g = 0; g < G; ++g) {
      const float m = stat[g], denom = stat[8 + g];
#pragma unroll 1
      for (int i = wtid; i < cl; i += kWorkers) sc[g * chunk + i] = bf16_round(expf(sc[g * chunk + i] - m) / denom);
    }
    // --- value sums, tile by tile
    float vacc[4][4];  // D[16 dims][query heads] of up to four dimension tiles of this warp's KV head
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) vacc[i][e] = 0.f;
    // --- value sums, pipelined like the scores.  The block meets once before the first tile (the
    // probabilities are complete) and in the tiles that are written by hand (new row, zeroed tail).
    named_bar_sync(1, kWorkers);
#pragma unroll 1
    for (int s = nt; s < 2 * nt; ++s) {
      const int t0 = j0 + (s - nt) * tile_keys, t1 = min(j1, t0 + tile_keys);
      uint8_t* tile = tiles + stage_of(s) * stage_bytes;
      tiles_ok = landed(s) && tiles_ok;
      const int tk = t1 - t0;
      const bool has_new = newpos >= t0 && newpos < t1, short_tile = (tk & 15) != 0;
      if (has_new || short_tile) {
        if (has_new) patch(tile, vn, newpos - t0);  // the new value rows join their tile
        if (short_tile) {
          // the last 16-key block of a short tile: rows past the tile's keys meet zero probabilities, but what
          // the stage holds there must be finite for that product to be zero
          const int count = 16 - (tk & 15), per_row = hpu * lpk;
          for (int it = wtid; it < count * per_row; it += kWorkers) {
            const int r = tk + it / per_row, rest = it % per_row;
            *reinterpret_cast<uint4*>(tile + piece_at(0u, rest / lpk, r, rest % lpk)) = make_uint4(0, 0, 0, 0);
          }
        }
        fence_proxy_async_all();
        named_bar_sync(1, kWorkers);
      }
      const uint32_t stage = smem_u32(tile);
      const float* pr = sc + (my_head * gs + lg) * chunk + (t0 - j0);
#pragma unroll 1
      for (int k16 = 0; k16 * 16 < tk; ++k16) {
        // B fragment: probabilities of query head lane / 4 for keys 2 * (lane % 4) + {0, 1} and + 8 of the block
        const int key = k16 * 16 + lt * 2;
        float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
        if (lg < gs) {
          if (key < tk) p0 = pr[key];
          if (key + 1 < tk) p1 = pr[key + 1];
          if (key + 8 < tk) p2 = pr[key + 8];
          if (key + 9 < tk) p3 = pr[key + 9];
        }
        const uint32_t b0 = pack2(p0, p1), b1 = pack2(p2, p3);
        // A fragment: V^T, from rows (keys) of the tile: matrices (keys 0-7 | 8-15) x (dims 0-7 | 8-15) of the block
        const int row = k16 * 16 + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int dt = my_slot + i * head_warps;
          if (dt < dim_tiles) {
            uint32_t af[4];
            ldmatrix_x4_trans(af, piece_at(stage, my_head, row, dt * 2 + ((lane >> 3) & 1)));
            mma_bf16_16816(vacc[i], af, b0, b1);
          }
        }
      }
      release(s);
    }
    trace_event(cx, wtid, EV_ATT_VALUES);
    if (!workers_ok(cx, tiles_ok)) {
      // a tile never came (or the launch was aborted elsewhere): the producer issues nothing more once it sees the
      // abort flag; what it had issued lands within a few microseconds, and the CTA stays for thirty
      for (int i = 0; i < 32; ++i) __nanosleep(1000);
      return false;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int dt = my_slot + i * head_warps;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = lt * 2 + (e & 1), d = dt * 16 + lg + (e >> 1) * 8;
        if (dt < dim_tiles && n < gs) red[(my_head * gs + n) * hd + d] = vacc[i][e];
      }
    }
    named_bar_sync(1, kWorkers);
#pragma unroll 1
    for (int col = wtid; col < cols; col += kWorkers) {
      const float o = red[col];
      const int g = col / hd, d = col - g * hd;
      const int head = kvh0 * gs + g;
      if (nch == 1) {
        A.out[b * A.out_bstride + head * A.out_hstride + d] = __float2bfloat16_rn(o);
      } else {
        const size_t row = static_cast<size_t>(b) * p.q_heads + head;
        __stcg(p.att_part + (row * kMaxChunks + ch) * hd + d, o);
      }
    }
    trace_event(cx, wtid, EV_ATT_PARTIAL);
    if (nch > 1 && A.combine) {
      // There is no consumer phase that adds chunk partials: chunk 0's CTA waits for the partials of its
      // peers (second stamp) and sums them in chunk order.
      float* mine = p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + ch) * kExchangeFloats;
      __threadfence();
      named_bar_sync(1, kWorkers);
      if (wtid == 0) st_relaxed_u32(reinterpret_cast<uint32_t*>(mine + kXchPartsFlag), A.stamp);
      if (ch == 0) {
        bool ok = true;
        if (wtid < nch) {
          const uint32_t* theirs = reinterpret_cast<const uint32_t*>(
              p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + wtid) * kExchangeFloats + kXchPartsFlag);
          uint32_t spins = 0;
          while (ld_relaxed_u32(theirs) != A.stamp) {
            if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, rowg)) {
              ok = false;
              break;
            }
          }
          __threadfence();
        }
        if (!workers_ok(cx, ok)) {
          cp_async_wait_all();
          return false;
        }
        for (int idx = wtid; idx < cols; idx += kWorkers) {
          const int g = idx / hd, d = idx - g * hd;
          const int head = kvh0 * gs + g;
          const size_t row = static_cast<size_t>(b) * p.q_heads + head;
          float o = 0.f;
          for (int c = 0; c < nch; ++c) o += __ldcg(p.att_part + (row * kMaxChunks + c) * hd + d);
          A.out[b * A.out_bstride + head * A.out_hstride + d] = __float2bfloat16_rn(o);
        }
      }
    }
    gtile += 2 * nt;
  }
  if (wtid == 0) cx.tc->kv_seq = gtile;  // read again after the barrier that closes this phase
  return true;
}

// Prompt attention (megabake::attention and the prefill pass) on the warp-level tensor cores.
//
// A unit is (sequence, query head, block of 64 query tokens).  The eight worker warps are four row
// groups of 16 query rows times two key halves: warps w and w + 4 keep the same q fragments in registers
// and split every 64-position K / V tile between them (positions 0-31 and 32-63), which halves the
// instruction chain of a tile; their statistics meet in shared memory after the first pass, their value
// sums after the second.  Tiles of the unit's KV head stream through the (idle) weight ring, two stages
// deep: the copies of the next tile are in flight while this one is multiplied, one block barrier per
// tile.  Two passes over the key tiles reproduce the reference's rounding points
// (src/megabake/lowering.py:274-300, the Hugging Face eager form): score = bf16(bf16(q.k) * scale)
// (+ additive mask, rounded again); softmax in fp32 against the row's global maximum and sum; probability
// rounded to bf16; fp32 value sums rounded once.
//   pass 1: scores of every tile -> running row maximum and sum of exp (rescaled when the maximum grows);
//   pass 2: the same scores again (same instructions, same bits) -> p = bf16(exp(s - max) / sum), which is
//           already the A-fragment layout of the next product, times the V tile (ldmatrix.trans).
// Without a mask tensor attention is causal: key j <= query token index, tiles past the block's last
// query are skipped, and so are the halves a warp's rows cannot see.  Causal blocks cost in proportion to
// their index, so the units are dealt heaviest first, every second round in reverse CTA order.  Rounded
// scores are bf16, so recomputing them costs tensor-core time only; no score buffer limits the key
// count.  One instantiation per head size: the fragment arrays then have their exact extents.
constexpr int kPromptQueries = 64;  // query rows per unit
constexpr int kPromptKeys = 64;     // positions per K / V tile

__device__ __forceinline__ uint32_t ldcg_u32(const void* ptr) { return __ldcg(reinterpret_cast<const unsigned int*>(ptr)); }

template <int HD>
__device__ __noinline__ bool attention_prompt(const Ctx& cx, const AttnArgs& A_in, int wtid) {
  // Private copies of the arguments and of the parameters this phase reads: every copy wait and block
  // barrier below is a compiler barrier for memory, behind which a value that lives behind a reference is
  // loaded again (a kernel parameter through the context: two dependent loads).
  const AttnArgs A = A_in;
  const int q_heads = cx.p->q_heads, kv_heads = cx.p->kv_heads, batch = cx.p->batch;
  const int my_cta = cx.cta, grid = cx.grid;
  constexpr int hd = HD;
  constexpr int ksteps = HD / 16;     // k steps of the score product
  constexpr int dtiles = HD / 8;      // 8-column tiles of the output row
  constexpr int pitch = HD * 2 + 16;  // bytes per tile row: 16 bytes of padding keep fragment loads conflict-free
  constexpr int pieces = HD / 8;      // 16-byte pieces per row
  constexpr int kStage = 2 * kPromptKeys * pitch;  // a K tile and a V tile
  constexpr int kStatFloats = 2 * 4 * 4 * 32;      // [key half][row group][m0, l0, m1, l1][lane]
  constexpr int kSumFloats = 4 * dtiles * 4 * 32;  // [row group][output element of a lane][lane]
  static_assert(2 * kStage + (kStatFloats + kSumFloats) * 4 <= kRingBytes, "prompt attention exceeds the weight ring");
  const int gs = q_heads / kv_heads;
  const int warp = wtid >> 5, lane = wtid & 31, g = lane >> 2, t = lane & 3;
  const int rw = warp & 3, kh = warp >> 2;  // row group, key half
  const int qblocks = (A.sq + kPromptQueries - 1) / kPromptQueries;
  const int heads = batch * q_heads;
  const int units = heads * qblocks;
  const uint32_t ring = smem_u32(cx.smem_a);
  float* const stat_x = reinterpret_cast<float*>(cx.smem_a + 2 * kStage);
  float* const sum_x = stat_x + kStatFloats;

#pragma unroll 1
  for (int round = 0; round * grid < units; ++round) {
    // heaviest first: sorted position i holds query block qblocks - 1 - i / heads
    const int i = round * grid + ((round & 1) ? grid - 1 - my_cta : my_cta);
    if (i >= units) continue;
    const int qb = qblocks - 1 - i / heads, bh = i % heads;
    const int h = bh % q_heads, b = bh / q_heads, kvh = h / gs;
    const int q0 = qb * kPromptQueries + rw * 16;
    const int r0 = q0 + g, r1 = r0 + 8;  // this thread's two query rows
    const int r0c = min(r0, A.sq - 1), r1c = min(r1, A.sq - 1);
    const bf16* qrow0 = A.q + b * A.q_bstride + static_cast<long long>(r0c) * A.q_ld + h * hd;
    const bf16* qrow1 = A.q + b * A.q_bstride + static_cast<long long>(r1c) * A.q_ld + h * hd;
    uint32_t qf[ksteps][4];
#pragma unroll
    for (int ks = 0; ks < ksteps; ++ks) {
      qf[ks][0] = ldcg_u32(qrow0 + ks * 16 + t * 2);
      qf[ks][1] = ldcg_u32(qrow1 + ks * 16 + t * 2);
      qf[ks][2] = ldcg_u32(qrow0 + ks * 16 + 8 + t * 2);
      qf[ks][3] = ldcg_u32(qrow1 + ks * 16 + 8 + t * 2);
    }
    const bf16* kbase = A.k + b * A.kv_bstride + kvh * hd;
    const bf16* vbase = A.v + b * A.kv_bstride + kvh * hd;
    const bf16* mrow0 = A.mask ? A.mask + (static_cast<long long>(b) * A.sq + r0c) * A.klen : nullptr;
    const bf16* mrow1 = A.mask ? A.mask + (static_cast<long long>(b) * A.sq + r1c) * A.klen : nullptr;
    const int kend = A.causal ? min(A.klen, qb * kPromptQueries + kPromptQueries) : A.klen;
    const int ntiles = (kend + kPromptKeys - 1) / kPromptKeys;
    const int steps = 2 * ntiles;  // pass 1 over the K tiles, then pass 2 over the K and V tiles

    // Step s copies into stage s & 1: the K tile, and in the second pass the V tile behind it.
    auto issue = [&](int s) {
      const bool second = s >= ntiles;
      const int j0 = (second ? s - ntiles : s) * kPromptKeys;
      const uint32_t ks_addr = ring + (s & 1) * kStage, vs_addr = ks_addr + kPromptKeys * pitch;
#pragma unroll
      for (int it0 = 0; it0 < kPromptKeys * pieces; it0 += kWorkers) {
        const int it = it0 + wtid;
        const int r = it / pieces, piece = it % pieces;
        const long long j = min(j0 + r, A.klen - 1);  // rows past the last key repeat it; they are masked below
        cp_async16(ks_addr + r * pitch + piece * 16, reinterpret_cast<const uint4*>(kbase + j * A.kv_ld) + piece);
        if (second) cp_async16(vs_addr + r * pitch + piece * 16, reinterpret_cast<const uint4*>(vbase + j * A.kv_ld) + piece);
      }
    };
    // Wait for step s's tile, then start the next step's copies into the stage every warp has just left.
    auto advance = [&](int s) {
      cp_async_wait_all();
      named_bar_sync(1, kWorkers);
      if (s + 1 < steps) issue(s + 1);
    };
    // Scores of this thread's two rows against keys j0 + nt * 8 + 2t, + 1 of the tile at ks_addr.
    auto score_tile = [&](uint32_t ks_addr, int j0, int nt, float (&out)[4]) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t krow = ks_addr + (nt * 8 + g) * pitch + t * 4;
#pragma unroll
      for (int ks = 0; ks < ksteps; ++ks) mma_bf16_16816(acc, qf[ks], lds_u32(krow + ks * 32), lds_u32(krow + ks * 32 + 16));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + nt * 8 + t * 2 + (e & 1);
        const int qi = (e < 2) ? r0 : r1;
        float v = bf16_round(bf16_round(acc[e]) * A.scale);
        if (A.mask) v = bf16_round(v + ldg_bf16(((e < 2) ? mrow0 : mrow1) + min(j, A.klen - 1)));
        const bool valid = j < A.klen && (!A.causal || j <= qi);
        out[e] = valid ? v : -INFINITY;
      }
    };
    named_bar_sync(1, kWorkers);  // every warp is done with the previous unit's last tile and its exchange areas
    issue(0);
    trace_event(cx, wtid, EV_ATT_INPUTS);

    // pass 1: row maximum and sum of exp over this warp's half of every tile
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
#pragma unroll 1
    for (int s = 0; s < ntiles; ++s) {
      const int j0 = s * kPromptKeys;
      const uint32_t ks_addr = ring + (s & 1) * kStage;
      advance(s);
      if (A.causal && j0 + kh * 32 > q0 + 15) continue;  // no query of this warp sees its half (barriers stay uniform)
      float sv[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) score_tile(ks_addr, j0, kh * 4 + nt, sv[nt]);
      float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        t0 = fmaxf(t0, fmaxf(sv[nt][0], sv[nt][1]));
        t1 = fmaxf(t1, fmaxf(sv[nt][2], sv[nt][3]));
      }
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
      const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        if (n0 > -INFINITY) s0 += expf(sv[nt][0] - n0) + expf(sv[nt][1] - n0);
        if (n1 > -INFINITY) s1 += expf(sv[nt][2] - n1) + expf(sv[nt][3] - n1);
      }
      s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      if (n0 > -INFINITY) { l0 = l0 * expf(m0 - n0) + s0; m0 = n0; }
      if (n1 > -INFINITY) { l1 = l1 * expf(m1 - n1) + s1; m1 = n1; }
    }
    trace_event(cx, wtid, EV_ATT_SCORES);
    {  // the two key halves' statistics meet: both warps of a row group form the same (max, sum), half 0 first
      float* mine = stat_x + (kh * 4 + rw) * 4 * 32 + lane;
      mine[0] = m0; mine[32] = l0; mine[64] = m1; mine[96] = l1;
      named_bar_sync(1, kWorkers);
      const float* other = stat_x + ((kh ^ 1) * 4 + rw) * 4 * 32 + lane;
      const float om0 = other[0], ol0 = other[32], om1 = other[64], ol1 = other[96];
      const float am0 = kh ? om0 : m0, al0 = kh ? ol0 : l0, bm0 = kh ? m0 : om0, bl0 = kh ? l0 : ol0;
      const float am1 = kh ? om1 : m1, al1 = kh ? ol1 : l1, bm1 = kh ? m1 : om1, bl1 = kh ? l1 : ol1;
      m0 = fmaxf(am0, bm0);
      m1 = fmaxf(am1, bm1);
      l0 = (am0 > -INFINITY ? al0 * expf(am0 - m0) : 0.f) + (bm0 > -INFINITY ? bl0 * expf(bm0 - m0) : 0.f);
      l1 = (am1 > -INFINITY ? al1 * expf(am1 - m1) : 0.f) + (bm1 > -INFINITY ? bl1 * expf(bm1 - m1) : 0.f);
    }

    // pass 2: the same scores, 16 keys at a time -> probabilities (already A fragments) x V
    float o[dtiles][4];
#pragma unroll
    for (int d = 0; d < dtiles; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
#pragma unroll 1
    for (int s = ntiles; s < steps; ++s) {
      const int j0 = (s - ntiles) * kPromptKeys;
      const uint32_t ks_addr = ring + (s & 1) * kStage, vs_addr = ks_addr + kPromptKeys * pitch;
      advance(s);
      if (A.causal && j0 + kh * 32 > q0 + 15) continue;
#pragma unroll
      for (int k2 = 0; k2 < 2; ++k2) {
        const int kk = kh * 2 + k2;  // 16-key block of the tile
        float sv[2][4];
        score_tile(ks_addr, j0, kk * 2, sv[0]);
        score_tile(ks_addr, j0, kk * 2 + 1, sv[1]);
        float pr[2][4];
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float sc = sv[half][e];
            const float m = (e < 2) ? m0 : m1, l = (e < 2) ? l0 : l1;
            pr[half][e] = (sc > -INFINITY) ? expf(sc - m) / l : 0.f;
          }
        uint32_t pa[4];
        pa[0] = pack2(pr[0][0], pr[0][1]);
        pa[1] = pack2(pr[0][2], pr[0][3]);
        pa[2] = pack2(pr[1][0], pr[1][1]);
        pa[3] = pack2(pr[1][2], pr[1][3]);
#pragma unroll
        for (int d = 0; d < dtiles; d += 2) {
          uint32_t vb[4];
          // matrices: (keys kk*16 + 0..7, dims d*8..), (keys + 8, same dims), then the same two for dims (d+1)*8..
          ldmatrix_x4_trans(vb, vs_addr + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * pitch + (d + (lane >> 4)) * 16);
          mma_bf16_16816(o[d], pa, vb[0], vb[1]);
          mma_bf16_16816(o[d + 1], pa, vb[2], vb[3]);
        }
      }
    }
    trace_event(cx, wtid, EV_ATT_VALUES);
    // the second half's fp32 sums join the first half's, which rounds once and stores
    float* sums = sum_x + rw * dtiles * 4 * 32 + lane;
    if (kh == 1) {
#pragma unroll
      for (int d = 0; d < dtiles; ++d)
#pragma unroll
        for (int e = 0; e < 4; ++e) sums[(d * 4 + e) * 32] = o[d][e];
    }
    named_bar_sync(1, kWorkers);
    if (kh == 0) {
      // this thread's output elements: rows r0, r1; columns d * 8 + t * 2, + 1
#pragma unroll
      for (int d = 0; d < dtiles; ++d) {
#pragma unroll
        for (int e = 0; e < 4; ++e) o[d][e] += sums[(d * 4 + e) * 32];
        if (r0 < A.sq)
          *reinterpret_cast<uint32_t*>(A.out + b * A.out_bstride + static_cast<long long>(r0) * A.out_tstride + h * A.out_hstride +
                                       d * 8 + t * 2) = pack2(o[d][0], o[d][1]);
        if (r1 < A.sq)
          *reinterpret_cast<uint32_t*>(A.out + b * A.out_bstride + static_cast<long long>(r1) * A.out_tstride + h * A.out_hstride +
                                       d * 8 + t * 2) = pack2(o[d][2], o[d][3]);
      }
    }
  }
  return true;
}

__device__ __forceinline__ bool attention_phase(const Ctx& cx, const AttnArgs& A, int wtid) {
  if (!A.decode) return cx.p->head_dim == 64 ? attention_prompt<64>(cx, A, wtid) : attention_prompt<128>(cx, A, wtid);
  return decode_stream_ok(*cx.p, A, cx.grid) ? attention_decode_stream(cx, A, wtid) : attention_decode(cx, A, wtid);
}

// Prefill: rotate q and k of every token in place in the qkv buffer.  An item is eight adjacent
// pairs (i, i + head_dim / 2) of one head of one token: two 16-byte loads of the row, one each of the
// cosine and sine rows, two 16-byte stores.
__device__ __noinline__ void rope_phase(const Ctx& cx, int wtid) {
  const KParams& p = *cx.p;
  const int hd = p.head_dim, half = hd / 2, vecs = half / 8;
  const int heads = p.q_heads + p.kv_heads;  // q heads then k heads are contiguous in a qkv row
  const int per_token = heads * vecs, items = p.m * per_token;
  const int style = p.prefill_rope_style, qkv_ld = p.qkv_ld, max_positions = p.max_positions;
  bf16* const qkv = p.qkv;
  const bf16 *cos_t = p.cos_t, *sin_t = p.sin_t;
  const long long* const positions = p.pos;
  for (int it = cx.cta * kWorkers + wtid; it < items; it += cx.grid * kWorkers) {
    const int t = it / per_token, rest = it - t * per_token;
    const int h = rest / vecs, i = (rest - h * vecs) * 8;
    long long pos = positions[t];
    if (pos < 0 || pos >= max_positions) pos = 0;
    bf16* x = qkv + static_cast<size_t>(t) * qkv_ld + h * hd + i;
    float a[8], b[8], c[8], sn[8];
    unpack8(__ldcg(reinterpret_cast<const uint4*>(x)), a);
    unpack8(__ldcg(reinterpret_cast<const uint4*>(x + half)), b);
    unpack8(__ldg(reinterpret_cast<const uint4*>(cos_t + pos * hd + i)), c);
    unpack8(__ldg(reinterpret_cast<const uint4*>(sin_t + pos * hd + i)), sn);
#pragma unroll
    for (int e = 0; e < 8; ++e) rope_pair(a[e], b[e], c[e], sn[e], style, a[e], b[e]);
    *reinterpret_cast<uint4*>(x) = pack8(a);
    *reinterpret_cast<uint4*>(x + half) = pack8(b);
  }
}

// ---------------------------------------------------------------------------
// tensor parallel: the all-reduce behind o_proj and down_proj, inside the kernel
//
// Called by every CTA of every rank after the grid barrier that closes an EPI_TP projection: by
// then each rank's CTAs have stored their partial sums into every rank's exchange buffer and
// fenced them at system scope.  CTA 0 posts this rank's arrival stamp in every rank's flag block
// (one release store per peer); every CTA waits, with the usual bound, until all stamps have
// reached its own GPU's flag block, then the grid adds, for its share of the residual stream,
//     hidden = bf16(hidden + bf16(sum over ranks, in rank order, of the fp32 partial sums)),
// the same rounding as the single-GPU split-K path, identical bits on every rank.  A grid
// barrier closes it.  Only plain loads of this GPU's own memory and plain peer stores are used:
// no multicast, no TMA on peer memory.  Stamps count up monotonically over the life of the
// group; the two halves of the exchange buffers alternate, so a rank that is one all-reduce
// ahead never overwrites what a slower rank is still adding.
__device__ __noinline__ bool tp_allreduce(const Ctx& cx, WorkerState& ws, int wtid, int index) {
  const KParams& p = *cx.p;
  const uint32_t stamp = p.tp_epoch + static_cast<uint32_t>(index) + 1u;
  const int half = index & 1;
  if (cx.cta == 0 && wtid < p.tp_size)
    st_release_sys_u32(reinterpret_cast<uint32_t*>(p.tp_peer[wtid]) + p.tp_rank, stamp);
  bool ok = true;
  if (wtid < p.tp_size) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(p.tp_peer[p.tp_rank]) + wtid;
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys_u32(flag) - stamp) < 0) {
      if ((++spins & 255u) == 0 && give_up(cx, SITE_TP_FLAG, wtid)) {
        ok = false;
        break;
      }
    }
  }
  if (!workers_ok(cx, ok)) return false;
  const int row_vecs = p.hidden / 8;
  const int nvec = p.m * row_vecs;
  for (int v = cx.cta * kWorkers + wtid; v < nvec; v += cx.grid * kWorkers) {
    const int t = v / row_vecs, c = v - t * row_vecs;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int src = 0; src < p.tp_size; ++src) {
      const float4* part = reinterpret_cast<const float4*>(tp_slot(p, p.tp_rank, half, src) + static_cast<size_t>(t) * p.hidden) + c * 2;
      const float4 lo = __ldcg(part), hi = __ldcg(part + 1);
      acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
      acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
    }
    uint4* at = reinterpret_cast<uint4*>(p.hidden_buf + static_cast<size_t>(t) * p.hidden) + c;
    float f[8];
    unpack8(__ldcg(at), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = bf16_round(f[e] + bf16_round(acc[e]));
    __stcg(at, pack8(f));
  }
  return grid_barrier(cx, ws, wtid);
}

// ---------------------------------------------------------------------------
// outputs of a launch that the prologue refused, and the device-side greedy sampler

// A launch whose prologue found a bad id, position or a full cache does no work.  Its outputs are
// filled with NaN so that a caller who reads them before looking at the status cannot mistake
// uninitialised memory for logits (the reference raises at this point: src/megabake/lowering.py:229).
__device__ __noinline__ void refuse_outputs(const Ctx& cx, int bad, int tid, int nthreads) {
  const KParams& p = *cx.p;
  bf16* out = nullptr;
  long long count = 0;
  if (p.mode == MODE_DECODE || p.mode == MODE_PREFILL) {
    out = p.logits;
    count = static_cast<long long>(p.m) * p.vocab;
  } else if (p.mode == MODE_KVATT) {
    out = p.op_out;
    count = static_cast<long long>(p.batch) * p.q_heads * p.head_dim;
  }
  const bf16 nan = __ushort_as_bfloat16(0x7FC0);
  for (long long i = static_cast<long long>(cx.cta) * nthreads + tid; out != nullptr && i < count;
       i += static_cast<long long>(cx.grid) * nthreads)
    out[i] = nan;
  if (cx.cta == 0 && tid == 0) {
    if (atomicCAS(&cx.ctrl->status, 0, bad) == 0) {
      cx.ctrl->where = SITE_PROLOGUE;
      cx.ctrl->cta = 0;
      cx.ctrl->detail = 0;
      if (p.status_mirror) *p.status_mirror = bad;
    }
    if (p.sample && p.tokens_out)
      for (int t = 0; t < p.m; ++t) p.tokens_out[t] = -1;
  }
  // Keep the monotonic barrier counter consistent with what the host expects.
  if (tid == 0 && p.nbar > 0) atomicAdd(&cx.ctrl->barrier, static_cast<uint32_t>(p.nbar));
}

// Greedy token of every sequence of the launch, taken from the bf16 logits the lm_head phase has
// written (the caller has passed a grid barrier since): the largest value, the lowest index among
// equal ones, as torch.argmax on the host would return.  CTA t serves token t.  The token goes to
// tokens_out[t] and becomes the next launch's id; the position moves on by one.  The kCount calling
// threads synchronise on named barrier kBarrier; `scratch` holds 64 words of shared memory.
template <int kBarrier, int kCount>
__device__ __noinline__ void greedy_sample(const Ctx& cx, int wtid, float* scratch) {
  const KParams& p = *cx.p;
  constexpr int nthreads = kCount;
  auto sync = [] { named_bar_sync(kBarrier, kCount); };
  const int lane = wtid & 31, warp = wtid >> 5, nwarps = nthreads >> 5;
  int* scratch_idx = reinterpret_cast<int*>(scratch + 32);
  for (int t = cx.cta; t < p.m; t += cx.grid) {
    const bf16* row = p.logits + static_cast<size_t>(t) * p.vocab;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    if ((p.vocab & 7) == 0) {
      const uint4* vrow = reinterpret_cast<const uint4*>(row);
      for (int v = wtid; v < p.vocab / 8; v += nthreads) {
        float f[8];
        unpack8(__ldcg(vrow + v), f);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (f[e] > best) { best = f[e]; idx = v * 8 + e; }
      }
    } else {
      for (int i = wtid; i < p.vocab; i += nthreads) {
        const float f = ldcg_bf16(row + i);
        if (f > best) { best = f; idx = i; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    sync();  // the scratch of the previous token has been read
    if (lane == 0) { scratch[warp] = best; scratch_idx[warp] = idx; }
    sync();
    if (wtid == 0) {
      for (int w = 1; w < nwarps; ++w)
        if (scratch[w] > best || (scratch[w] == best && scratch_idx[w] < idx)) { best = scratch[w]; idx = scratch_idx[w]; }
      if (idx == 0x7fffffff) idx = 0;  // every logit NaN
      if (p.tokens_out) p.tokens_out[t] = idx;
      p.ids[t] = idx;
      p.pos[t] += 1;
    }
  }
}

// ---------------------------------------------------------------------------
// workers: whole-launch schedule

__device__ void worker_loop(const Ctx& cx, int wtid) {
  const KParams& p = *cx.p;
  WorkerState ws;
  ws.tiles = 0; ws.passed = 0;
  // A projection phase: publish its operand (complete since the last grid barrier), run the epilogues.
  auto gemm = [&](int gp) -> bool {
    signal_operand(cx, gp, wtid);
    return worker_gemm_tc(cx, gp, ws, wtid);
  };
  // A projection whose operand is the RMSNorm of the residual stream: normalise the rows first.
  auto normed_gemm = [&](int gp) -> bool {
    norm_phase(cx, &cx.misc->phase[gp & 1], wtid);
    if (!grid_barrier(cx, ws, wtid)) return false;
    return gemm(gp);
  };
  const int q_size = p.q_heads * p.head_dim, kv_size = p.kv_heads * p.head_dim;
  AttnArgs A;
  A.knew = nullptr; A.vnew = nullptr; A.new_ld = 0; A.mask = nullptr;
  A.sq = 1; A.klen = 0; A.len = 0; A.lens = nullptr; A.decode = 0; A.rope = 0; A.causal = 0; A.combine = 0;
  A.kmap = nullptr; A.vmap = nullptr;
  A.stamp = p.att_epoch + 1; A.scale = p.att_scale;
  if (p.n_gemm > 0) {
    prefetch_phase(cx, 0, wtid);
    named_bar_sync(1, kWorkers);
  }
  if (p.mode == MODE_LINEAR) {
    gemm(0);
    return;
  }
  if (p.mode == MODE_KVATT) {
    A.q = p.op_q; A.q_bstride = q_size; A.q_ld = q_size;
    A.k = static_cast<bf16*>(p.kc[0]); A.v = static_cast<bf16*>(p.vc[0]);
    A.kv_bstride = static_cast<long long>(p.capacity) * kv_size; A.kv_ld = kv_size;
    A.knew = p.op_k; A.vnew = p.op_v; A.new_ld = kv_size;
    A.out = p.op_out; A.out_bstride = q_size; A.out_tstride = 0; A.out_hstride = p.head_dim;
    A.len = *p.len[0]; A.lens = nullptr; A.decode = 1; A.combine = 1;
    if (!attention_phase(cx, A, wtid)) return;
    if (!grid_barrier(cx, ws, wtid)) return;
    if (cx.cta == 0 && wtid == 0) *p.len[0] = A.len + 1;
    return;
  }
  if (p.mode == MODE_ATT) {
    A.q = p.op_q; A.q_bstride = static_cast<long long>(p.op_qlen) * q_size; A.q_ld = q_size;
    A.k = const_cast<bf16*>(p.op_k); A.v = const_cast<bf16*>(p.op_v);
    A.kv_bstride = static_cast<long long>(p.op_klen) * kv_size; A.kv_ld = kv_size;
    A.out = p.op_out;  // [batch*heads, q_len, head_dim]
    A.out_bstride = static_cast<long long>(p.q_heads) * p.op_qlen * p.head_dim;
    A.out_tstride = p.head_dim; A.out_hstride = p.op_qlen * p.head_dim;
    A.mask = p.mask; A.sq = p.op_qlen; A.klen = p.op_klen;
    attention_phase(cx, A, wtid);
    return;
  }
  // Layer 0's residual stream starts as the embedding rows (the split-K table writes them from its first
  // normalising phase).  Its first reader is layer 0's o_proj epilogue, two grid barriers on.
  for (int v = cx.cta * kWorkers + wtid; !p.split && v < p.m * (p.hidden / 8); v += cx.grid * kWorkers) {
    const int t = v / (p.hidden / 8), c = v - t * (p.hidden / 8);
    long long id = p.ids[t];
    if (id < 0 || id >= p.embed_rows) id = 0;
    reinterpret_cast<uint4*>(p.hidden_buf + static_cast<size_t>(t) * p.hidden)[c] =
        __ldg(reinterpret_cast<const uint4*>(p.embed + id * p.hidden) + c);
  }
  const bool decode = (p.mode == MODE_DECODE);
  for (int layer = 0; layer < p.layers; ++layer) {
    if (!normed_gemm(layer * 4 + 0)) return;                // RMSNorm | q, k, v (+bias)
    if (!grid_barrier(cx, ws, wtid)) return;
    A.q = p.qkv; A.q_ld = p.qkv_ld;
    A.out = p.attn; A.out_tstride = q_size; A.out_hstride = p.head_dim;
    A.stamp = p.att_epoch + static_cast<uint32_t>(layer) + 1u;
    if (decode) {
      A.q_bstride = p.qkv_ld;
      A.k = static_cast<bf16*>(p.kc[layer]); A.v = static_cast<bf16*>(p.vc[layer]);
      A.kv_bstride = static_cast<long long>(p.capacity) * kv_size; A.kv_ld = kv_size;
      A.knew = p.qkv + q_size; A.vnew = A.knew + kv_size; A.new_ld = p.qkv_ld;
      A.out_bstride = q_size;
      if (p.ragged) {  // one valid length per sequence: the context split follows the longest
        A.lens = p.len[layer];
        int longest = 0;
        for (int b = 0; b < p.batch; ++b) longest = max(longest, A.lens[b]);
        A.len = longest;
      } else {
        A.len = *p.len[layer];
      }
      A.decode = 1; A.rope = 1;
      A.kmap = p.kv_maps ? p.kv_maps + layer : nullptr;
      A.vmap = p.kv_maps ? p.kv_maps + p.layers + layer : nullptr;
      A.combine = 1;  // the o projection fetches a finished bf16 matrix: the first chunk's CTA sums the chunk partials
    } else {
      rope_phase(cx, wtid);
      if (!grid_barrier(cx, ws, wtid)) return;
      A.q_bstride = static_cast<long long>(p.seq) * p.qkv_ld;
      A.k = p.qkv + q_size; A.v = A.k + kv_size;
      A.kv_bstride = static_cast<long long>(p.seq) * p.qkv_ld; A.kv_ld = p.qkv_ld;
      A.out_bstride = static_cast<long long>(p.seq) * q_size;
      A.mask = p.mask; A.sq = p.seq; A.klen = p.seq; A.causal = (p.mask == nullptr);
    }
    if (!attention_phase(cx, A, wtid)) return;              // [RoPE] attention (+ KV append); decode streams cache tiles through the ring
    named_bar_sync(1, kWorkers);                            // every worker is done with the ring
    if (wtid == 0) *reinterpret_cast<volatile int*>(&cx.tc->a_ready) = layer * 4 + 2;  // o_proj's weights may come
    trace_event(cx, wtid, EV_ATTENTION_DONE);
    if (!grid_barrier(cx, ws, wtid)) return;
    if (decode && cx.cta == 0) {  // publish after the interval closes
      if (p.ragged) {
        for (int b = wtid; b < p.batch; b += kWorkers) p.len[layer][b] = A.lens[b] + 1;
      } else if (wtid == 0) {
        *p.len[layer] = A.len + 1;
      }
    }
    if (!gemm(layer * 4 + 1)) return;                       // o_proj + residual (tensor parallel: partial sums to every rank)
    if (!grid_barrier(cx, ws, wtid)) return;
    if (p.tp_size > 1 && !tp_allreduce(cx, ws, wtid, 2 * layer)) return;
    if (!normed_gemm(layer * 4 + 2)) return;                // RMSNorm | gate, up -> SiLU*up
    if (!grid_barrier(cx, ws, wtid)) return;
    if (!gemm(layer * 4 + 3)) return;                       // down + residual
    if (!grid_barrier(cx, ws, wtid)) return;
    if (p.tp_size > 1 && !tp_allreduce(cx, ws, wtid, 2 * layer + 1)) return;
  }
  if (!normed_gemm(p.layers * 4)) return;                   // final RMSNorm | lm_head
  if (p.sample) {
    if (!grid_barrier(cx, ws, wtid)) return;                // every CTA's logits are out and nobody reads ids/positions any more
    greedy_sample<1, kWorkers>(cx, wtid, reinterpret_cast<float*>(cx.smem_b));
  }
}

// ---------------------------------------------------------------------------
// the kernel

__global__ void __launch_bounds__(kThreads, 1) megakernel(const __grid_constant__ KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctx cx;
  cx.p = &p;
  cx.ctrl = p.ctrl;
  cx.smem_a = smem;
  cx.smem_b = smem + kRingBytes;
  cx.misc = reinterpret_cast<SmemMisc*>(cx.smem_b + kBBytes);
  cx.tc = reinterpret_cast<SmemMiscTc*>(cx.smem_b + kBBytes + kMiscBytes);
  cx.deadline = clock64() + p.timeout_cycles;
  cx.cta = blockIdx.x;
  cx.grid = gridDim.x;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool tc = p.n_gemm > 0;   // tensor-core roles (TMEM, MMA issuer, the two producers)

  if (tid < kChunkBars) {  // one barrier quadruple per thread
    mbar_init(smem_u32(&cx.misc->full[tid]), 1);
    mbar_init(smem_u32(&cx.misc->empty[tid]), 1);   // one MMA commit
    mbar_init(smem_u32(&cx.tc->bfull[tid]), 1);
    mbar_init(smem_u32(&cx.tc->bempty[tid]), 1);
    mbar_fence_init();
  }
  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&cx.misc->accfull[b]), 1);
      mbar_init(smem_u32(&cx.misc->accempty[b]), kWorkers);
    }
    cx.misc->wabort = 0;
    cx.misc->bad = 0;
    cx.misc->flag = 0;
    cx.misc->trace_n = 0;
    cx.misc->trace_on = p.trace_cap != 0;
    cx.misc->n_gemm = p.n_gemm;
    cx.misc->epoch = p.epoch;
    cx.misc->phases = p.phases;
    cx.tc->b_ready = 0;
    cx.tc->a_ready = 0;
    cx.tc->kv_seq = 0;
    cx.tc->kv_req = 0;
    for (int st = 0; st < 8; ++st) {
      mbar_init(smem_u32(&cx.tc->kvfull[st]), 1);
      mbar_init(smem_u32(&cx.tc->kvempty[st]), kWorkerWarps);
    }
    mbar_fence_init();
    mbar_fence_init();
  }
  // The rows of a 128-row MMA tile that a weight copy does not fill hold whatever the ring held before;
  // they only ever reach accumulator rows that no epilogue reads, so the ring needs no clearing.
  __syncthreads();
  if (warp == 1 && tc) {
    tmem_alloc(smem_u32(&cx.misc->tmem_base), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }

  // Prologue validation: same inputs in every CTA, so the verdict is grid-uniform.
  if (p.mode == MODE_DECODE || p.mode == MODE_PREFILL || p.mode == MODE_KVATT) {
    int bad = 0;
    if (p.mode != MODE_KVATT) {
      for (int t = tid; t < p.m; t += kThreads) {
        const long long id = p.ids[t], pos = p.pos[t];
        if (id < 0 || id >= p.embed_rows || pos < 0 || pos >= p.max_positions) bad = MK_STATUS_BAD_INDEX;
      }
    }
    if (p.mode != MODE_PREFILL) {
      const int nl = (p.mode == MODE_KVATT) ? 1 : p.layers;
      const int per_layer = p.ragged ? p.batch : 1;
      for (int i = tid; i < nl * per_layer; i += kThreads) {
        const int len = p.len[i / per_layer][i % per_layer];
        if (len < 0 || len + 1 > p.capacity) bad = MK_STATUS_KV_OVERFLOW;
      }
    }
    if (bad) atomicMax(&cx.misc->bad, bad);
  }
  __syncthreads();
  tc_fence_after();
  const int bad = *reinterpret_cast<volatile int*>(&cx.misc->bad);
  if (bad) {
    refuse_outputs(cx, bad, tid, kThreads);
  } else if (warp == 0) {
    if (tc && tid == 0) producer_loop(cx);
  } else if (warp == 1) {
    if (tc && tid == 32) mma_loop(cx);
  } else if (warp <= 1 + kWorkerWarps) {
    worker_loop(cx, tid - 64);
  } else {
    if (tc && tid == 64 + kWorkers) activation_producer_loop(cx);
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1 && tc) {
    tc_fence_after();
    tmem_dealloc(*reinterpret_cast<volatile uint32_t*>(&cx.misc->tmem_base), kTmemCols);
  }
}

}  // namespace mk
