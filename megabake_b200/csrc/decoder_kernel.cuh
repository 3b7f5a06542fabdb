// The persistent decoder megakernel for sm_100a: one cooperative launch runs a
// whole Llama/Qwen2-style decoder step.
//
// Roles inside each CTA (one CTA per SM):
//   warp 0      weight producer: walks the static schedule of every projection
//               phase of the launch and streams this CTA's share of the weights
//               through a ring of TMA stages.  Weights never depend on a
//               barrier, so the stream runs ahead across phases and layers.
//   warp 1      MMA issuer: tcgen05.mma with the weight tile as the M=128
//               operand and the token activations as the N=16 operand
//               (the "swapAB" orientation), fp32 accumulators in TMEM.
//   warps 2-5   workers: build the activation operand in shared memory
//               (RMSNorm fused here), run the epilogues out of TMEM (bias,
//               residual add, SiLU*up), the attention phase (RoPE, KV append,
//               split-context softmax attention) and the grid barriers.
//
// Work split: each projection phase is flattened to 16 KiB weight chunks
// (128 rows x 64 K) in tile-major order and cut into equal contiguous ranges,
// one per CTA.  A tile whose K range spans several CTAs is finished by the
// last CTA to arrive, which sums the fp32 partials in CTA order (fixed order,
// so results do not depend on timing).
//
// Every device wait is bounded: a wait that runs out records where in the
// status block, raises the abort flag that all other waits poll, and the CTA
// leaves through the common exit (drain TMA, free TMEM).  Nothing traps.
#pragma once
#include "megakernel.cuh"
#include "ptx.cuh"

namespace mk {

struct SmemMisc {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t accfull[2];
  uint64_t accempty[2];
  uint64_t bfull;
  uint32_t tmem_base;
  int wabort;  // sticky: a worker thread gave up a wait
  int bad;     // prologue validation result
  int flag;    // "this CTA reduces / finishes" decisions taken by worker thread 0
  float rinv[kTok];
  int trace_n;  // events this CTA has recorded
};
static_assert(sizeof(SmemMisc) <= kMiscBytes, "misc shared block too large");

struct Ctx {
  const KParams* p;
  Control* ctrl;
  SmemMisc* misc;
  uint8_t* smem_a;
  uint8_t* smem_b;
  long long deadline;
  int cta, grid;
};

struct Range {
  long long c0, c1;
  int geff;
};

// ---------------------------------------------------------------------------
// bounded waits

__device__ __noinline__ bool give_up(const Ctx& cx, int site, int detail) {
  if (ld_relaxed_u32(&cx.ctrl->abort) != 0) return true;
  if (clock64() > cx.deadline) {
    if (atomicCAS(&cx.ctrl->status, 0, static_cast<int>(MK_STATUS_TIMEOUT)) == 0) {
      cx.ctrl->where = site;
      cx.ctrl->cta = cx.cta;
      cx.ctrl->detail = detail;
    }
    atomicExch(&cx.ctrl->abort, 1u);
    __threadfence();
    return true;
  }
  return false;
}

// Optional per-CTA event trace (worker thread 0 only): what the reference's
// MEGABAKE_PHASE_TIMER stamps give (src/megabake/runtime.py:27-46).
__device__ __forceinline__ void trace_event(const Ctx& cx, int wtid, int code) {
  if (cx.p->trace_cap == 0 || wtid != 0) return;
  const int n = cx.misc->trace_n;
  if (n >= cx.p->trace_cap) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  cx.p->trace[static_cast<size_t>(cx.cta) * cx.p->trace_cap + n] =
      (static_cast<unsigned long long>(code) << 56) | (t & 0x00FFFFFFFFFFFFFFull);
  cx.misc->trace_n = n + 1;
}

__device__ __forceinline__ bool wait_mbar(const Ctx& cx, uint32_t bar, uint32_t parity, int site, int detail) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0 && give_up(cx, site, detail)) return false;
  }
  return true;
}

// Worker-uniform decision: true only if no worker thread has given up.
__device__ __forceinline__ bool workers_ok(const Ctx& cx, bool ok) {
  if (!ok) cx.misc->wabort = 1;
  named_bar_sync(1, kWorkers);
  return *reinterpret_cast<volatile int*>(&cx.misc->wabort) == 0;
}

// Monotonic-counter grid barrier over the worker warps of every CTA: one
// release-add to arrive, relaxed polling, one fence once the count is reached.
__device__ bool grid_barrier(const Ctx& cx, uint32_t& passed, int wtid) {
  named_bar_sync(1, kWorkers);
  passed += 1;
  if (wtid == 0) {
    red_release_add_u32(&cx.ctrl->barrier, 1u);
    const uint32_t target = cx.p->epoch + passed * static_cast<uint32_t>(cx.grid);
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_relaxed_u32(&cx.ctrl->barrier) - target) < 0) {
      if ((++spins & 255u) == 0 && give_up(cx, SITE_GRID_BARRIER, static_cast<int>(passed))) {
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
// work split

__device__ __forceinline__ Range cta_range(const GemmPhase* ph, int cta, int grid) {
  Range r;
  const long long total = ph->total;
  r.geff = total < grid ? static_cast<int>(total) : grid;
  if (cta >= r.geff) {
    r.c0 = r.c1 = 0;
    return r;
  }
  r.c0 = cta * total / r.geff;
  r.c1 = (cta + 1) * total / r.geff;
  return r;
}

__device__ __forceinline__ int cta_of_chunk(long long chunk, long long total, int geff) {
  return static_cast<int>(((chunk + 1) * geff + total - 1) / total) - 1;
}

__device__ __forceinline__ int segment_of_tile(const GemmPhase* ph, int tile) {
  int seg = 0;
  while (seg + 1 < ph->nseg && tile >= ph->tile_start[seg + 1]) ++seg;
  return seg;
}

// ---------------------------------------------------------------------------
// warp 0: weight producer

__device__ __noinline__ void producer_loop(const Ctx& cx) {
  const KParams& p = *cx.p;
  const uint64_t policy = p.stream_once ? l2_policy_evict_first() : l2_policy_evict_normal();
  const int ntt = (p.m + kTok - 1) / kTok;
  uint32_t it = 0;
  bool ok = true;
  for (int gp = 0; gp < p.n_gemm && ok; ++gp) {
    const GemmPhase* ph = p.phases + gp;
    const Range r = cta_range(ph, cx.cta, cx.grid);
    if (r.c1 <= r.c0) continue;
    const int tc = ph->tc, nacc = ph->nacc;
    for (int tt = 0; tt < ntt && ok; ++tt) {
      long long c = r.c0;
      while (c < r.c1 && ok) {
        const int tile = static_cast<int>(c / tc);
        long long seg_end = static_cast<long long>(tile + 1) * tc;
        if (seg_end > r.c1) seg_end = r.c1;
        const CUtensorMap* map0 = ph->tmap[0];
        int row0 = tile * kTileRows;
        if (nacc == 1) {
          const int seg = segment_of_tile(ph, tile);
          map0 = ph->tmap[seg];
          row0 = (tile - ph->tile_start[seg]) * kTileRows;
        }
        for (; c < seg_end; ++c) {
          const int j = static_cast<int>(c - static_cast<long long>(tile) * tc);
          const int kidx = j / nacc;
          const CUtensorMap* map = (nacc == 2) ? ph->tmap[j % nacc] : map0;
          const uint32_t stage = it % kStages;
          const uint32_t parity = (it / kStages) & 1u;
          if (!wait_mbar(cx, smem_u32(&cx.misc->empty[stage]), parity ^ 1u, SITE_PRODUCER_EMPTY, gp)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&cx.misc->full[stage]);
          mbar_expect_tx(full, kStageBytes);
          tma_load_2d(smem_u32(cx.smem_a + stage * kStageBytes), map, kidx * kChunkK, row0, full, policy);
          ++it;
        }
      }
    }
  }
  if (!ok) {
    // Leaving early: every copy already issued must land before the CTA exits.
    const uint32_t first = it > kStages ? it - kStages : 0;
    for (uint32_t i = first; i < it; ++i) {
      const uint32_t bar = smem_u32(&cx.misc->full[i % kStages]);
      for (uint32_t spins = 0; spins < (1u << 22); ++spins) {
        if (mbar_try_wait(bar, (i / kStages) & 1u)) break;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// warp 1: MMA issuer

__device__ __noinline__ void mma_loop(const Ctx& cx) {
  const KParams& p = *cx.p;
  const int ntt = (p.m + kTok - 1) / kTok;
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&cx.misc->tmem_base);
  constexpr uint32_t idesc = umma_idesc_bf16(kTileRows, kTok);
  uint32_t it = 0, q = 0, bcount = 0;
  for (int gp = 0; gp < p.n_gemm; ++gp) {
    const GemmPhase* ph = p.phases + gp;
    const Range r = cta_range(ph, cx.cta, cx.grid);
    if (r.c1 <= r.c0) continue;
    const int tc = ph->tc, nacc = ph->nacc, kc = ph->kc;
    const long long ks0 = r.c0 / nacc;
    const long long ks1 = (r.c1 + nacc - 1) / nacc;
    const bool all_k = (ks1 - ks0) >= kc;
    for (int tt = 0; tt < ntt; ++tt) {
      if (!wait_mbar(cx, smem_u32(&cx.misc->bfull), bcount & 1u, SITE_MMA_B, gp)) return;
      ++bcount;
      tc_fence_after();
      long long c = r.c0;
      while (c < r.c1) {
        const int tile = static_cast<int>(c / tc);
        long long seg_end = static_cast<long long>(tile + 1) * tc;
        if (seg_end > r.c1) seg_end = r.c1;
        const uint32_t buf = q & 1u;
        if (!wait_mbar(cx, smem_u32(&cx.misc->accempty[buf]), ((q >> 1) & 1u) ^ 1u, SITE_MMA_ACC, gp)) return;
        tc_fence_after();
        uint32_t started0 = 0, started1 = 0;
        for (; c < seg_end; ++c) {
          const int j = static_cast<int>(c - static_cast<long long>(tile) * tc);
          const int kidx = j / nacc;
          const int acc = j - kidx * nacc;
          const int slot = all_k ? kidx : static_cast<int>(c / nacc - ks0);
          const uint32_t stage = it % kStages;
          if (!wait_mbar(cx, smem_u32(&cx.misc->full[stage]), (it / kStages) & 1u, SITE_MMA_FULL, gp)) return;
          tc_fence_after();
          const uint32_t a_base = smem_u32(cx.smem_a + stage * kStageBytes);
          const uint32_t b_base = smem_u32(cx.smem_b + slot * kBSlotBytes);
          const uint32_t d = tmem + (buf * 2u + static_cast<uint32_t>(acc)) * kTok;
          uint32_t started = acc ? started1 : started0;
#pragma unroll
          for (int kk = 0; kk < kChunkK / 16; ++kk) {
            umma_bf16(d, umma_desc_sw128(a_base + kk * 32), umma_desc_sw128(b_base + kk * 32), idesc,
                      started | static_cast<uint32_t>(kk > 0));
          }
          if (acc) started1 = 1; else started0 = 1;
          umma_commit(smem_u32(&cx.misc->empty[stage]));
          ++it;
        }
        umma_commit(smem_u32(&cx.misc->accfull[buf]));
        ++q;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// workers: activation operand staging

__device__ __forceinline__ const bf16* activation_row(const KParams& p, const GemmPhase* ph, int token) {
  if (ph->gather) {
    long long id = p.ids[token];
    if (id < 0 || id >= p.vocab) id = 0;  // reported by the prologue; never dereference out of range
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

// RMSNorm statistics of the rows of one token tile: rinv[t] = 1/sqrt(mean(x^2)+eps).
// One warp per token; eight 16-byte loads are in flight per lane before any is used.
__device__ __noinline__ void norm_stats(const Ctx& cx, const GemmPhase* ph, int t0, int mt, int wtid) {
  const KParams& p = *cx.p;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int nvec = p.hidden / 8;
  for (int t = warp; t < mt; t += kWorkerWarps) {
    const uint4* row = reinterpret_cast<const uint4*>(activation_row(p, ph, t0 + t));
    float sum = 0.f;
    for (int v0 = 0; v0 < nvec; v0 += 32 * 8) {
      uint4 u[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int v = v0 + i * 32 + lane;
        u[i] = v < nvec ? __ldcg(row + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float f[8];
        unpack8(u[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) sum = fmaf(f[e], f[e], sum);
      }
    }
    sum = warp_sum(sum);
    if (lane == 0) cx.misc->rinv[t] = 1.0f / sqrtf(sum / static_cast<float>(p.hidden) + p.eps);
  }
  named_bar_sync(1, kWorkers);
}

// Normalise one 8-element vector: w * bf16(x * rinv), the two roundings of the
// Hugging Face RMSNorm.
__device__ __forceinline__ uint4 normalise_vec(const uint4& xu, const uint4& wu, float r) {
  float x[8], w[8];
  unpack8(xu, x);
  unpack8(wu, w);
#pragma unroll
  for (int e = 0; e < 8; ++e) x[e] = w[e] * bf16_round(x[e] * r);
  return pack8(x);
}

// One 8-element vector of the activation operand (normalised if the phase asks).
__device__ __forceinline__ uint4 activation_vec(const Ctx& cx, const GemmPhase* ph, const bf16* row, int t, int col) {
  const uint4 u = __ldcg(reinterpret_cast<const uint4*>(row + col));
  if (ph->bmode != B_NORM) return u;
  return normalise_vec(u, __ldg(reinterpret_cast<const uint4*>(ph->normw + col)), cx.misc->rinv[t]);
}

// Fill the swizzled (SWIZZLE_128B, K-major) activation slots this CTA's chunk
// range needs.  Loads are issued four at a time per thread before any is used.
__device__ __noinline__ void stage_b(const Ctx& cx, const GemmPhase* ph, const Range& r, int t0, int mt, int wtid) {
  const KParams& p = *cx.p;
  const bool norm = ph->bmode == B_NORM;
  if (norm) norm_stats(cx, ph, t0, mt, wtid);
  const int nacc = ph->nacc, kc = ph->kc;
  const long long ks0 = r.c0 / nacc;
  const long long ks1 = (r.c1 + nacc - 1) / nacc;
  const bool all_k = (ks1 - ks0) >= kc;
  const int nk = all_k ? kc : static_cast<int>(ks1 - ks0);
  const int per_slot = mt * 8;
  const int items = nk * per_slot;
  const bf16* normw = ph->normw;
  for (int item0 = wtid; item0 < items; item0 += kWorkers * 4) {
    uint4 xu[4], wu[4];
    int slot[4], tok[4], vec[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int item = item0 + i * kWorkers;
      if (item < items) {
        slot[i] = item / per_slot;
        const int rem = item - slot[i] * per_slot;
        tok[i] = rem >> 3;
        vec[i] = rem & 7;
        const int kidx = all_k ? slot[i] : static_cast<int>((ks0 + slot[i]) % kc);
        const int col = kidx * kChunkK + vec[i] * 8;
        xu[i] = __ldcg(reinterpret_cast<const uint4*>(activation_row(p, ph, t0 + tok[i]) + col));
        if (norm) wu[i] = __ldg(reinterpret_cast<const uint4*>(normw + col));
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int item = item0 + i * kWorkers;
      if (item < items) {
        const uint4 u = norm ? normalise_vec(xu[i], wu[i], cx.misc->rinv[tok[i]]) : xu[i];
        uint8_t* dst = cx.smem_b + slot[i] * kBSlotBytes + (tok[i] >> 3) * 1024 + (tok[i] & 7) * 128 +
                       ((vec[i] ^ (tok[i] & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = u;
      }
    }
  }
  fence_proxy_async_smem();
  mbar_arrive(smem_u32(&cx.misc->bfull));
}

// ---------------------------------------------------------------------------
// workers: epilogues

__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

__device__ void apply_epilogue(const Ctx& cx, const GemmPhase* ph, int tile, int rloc, float (*v)[kTok], int t0,
                               int mt) {
  const KParams& p = *cx.p;
  if (ph->nacc == 2) {
    const int n = tile * kTileRows + rloc;
    if (n >= ph->n[0]) return;
    for (int t = 0; t < mt; ++t) {
      const float gate = bf16_round(v[0][t]);
      const float up = bf16_round(v[1][t]);
      const float act = bf16_round(silu(gate));
      ph->dst[static_cast<size_t>(t0 + t) * ph->dst_ld + n] = __float2bfloat16_rn(act * up);
    }
    return;
  }
  const int seg = segment_of_tile(ph, tile);
  const int n = (tile - ph->tile_start[seg]) * kTileRows + rloc;
  if (n >= ph->n[seg]) return;
  bf16* dst = ph->to_logits ? p.logits : ph->dst;
  const size_t col = static_cast<size_t>(ph->out_col[seg]) + n;
  if (ph->epi == EPI_STORE) {
    const float bias = ph->bias[seg] ? ldg_bf16(ph->bias[seg] + n) : 0.f;
    for (int t = 0; t < mt; ++t)
      dst[static_cast<size_t>(t0 + t) * ph->dst_ld + col] = __float2bfloat16_rn(v[0][t] + bias);
  } else {  // EPI_RESIDUAL: hidden += bf16(projection), in place
    for (int t = 0; t < mt; ++t) {
      bf16* h = dst + static_cast<size_t>(t0 + t) * ph->dst_ld + col;
      const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(h));
      const float residual = __bfloat162float(__ushort_as_bfloat16(raw));
      *h = __float2bfloat16_rn(residual + bf16_round(v[0][t]));
    }
  }
}

// Split-K completion for one tile segment.  The CTA that holds the tile's first
// chunk reduces: for it the tile is the last segment of its range, so by then
// the other contributors (for which the tile comes first) have published their
// fp32 partials.  Contributors store, fence, count themselves and move on; the
// reducer waits (bounded) for the count, then adds the partials to its own
// accumulators in CTA order, which fixes the summation order.
__device__ __noinline__ bool finish_split(const Ctx& cx, const GemmPhase* ph, const Range& r, int tile, int rloc,
                             float (*v)[kTok], int t0, int mt, int wtid) {
  const KParams& p = *cx.p;
  const int tc = ph->tc, nacc = ph->nacc;
  const long long total = ph->total;
  const int first = cta_of_chunk(static_cast<long long>(tile) * tc, total, r.geff);
  const int last = cta_of_chunk(static_cast<long long>(tile + 1) * tc - 1, total, r.geff);
  if (cx.cta != first) {
    const int slot = (static_cast<int>(r.c0 / tc) == tile) ? 0 : 1;
    float* mine = p.partials + static_cast<size_t>(cx.cta * 2 + slot) * kPartialFloats;
    for (int a = 0; a < nacc; ++a)
      for (int t = 0; t < mt; ++t) __stcg(mine + (a * kTok + t) * kTileRows + rloc, v[a][t]);
    __threadfence();
    named_bar_sync(1, kWorkers);
    if (wtid == 0) red_release_add_u32(&p.tile_ctr[tile], 1u);
    return true;
  }
  if (wtid == 0) {
    const uint32_t expected = static_cast<uint32_t>(last - first);
    uint32_t spins = 0;
    while (ld_relaxed_u32(&p.tile_ctr[tile]) < expected) {
      if ((++spins & 255u) == 0 && give_up(cx, SITE_SPLIT_REDUCE, tile)) {
        cx.misc->wabort = 1;
        break;
      }
    }
    p.tile_ctr[tile] = 0;  // the next use is behind a grid barrier
    __threadfence();
  }
  named_bar_sync(1, kWorkers);
  if (*reinterpret_cast<volatile int*>(&cx.misc->wabort)) return false;
  for (int g0 = first + 1; g0 <= last; g0 += 4) {
    float part[4][2];
    for (int t = 0; t < mt; ++t) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int g = g0 + i;
        if (g <= last) {
          const int gslot = (static_cast<int>((g * total / r.geff) / tc) == tile) ? 0 : 1;
          const float* theirs = p.partials + static_cast<size_t>(g * 2 + gslot) * kPartialFloats;
          part[i][0] = __ldcg(theirs + t * kTileRows + rloc);
          if (nacc == 2) part[i][1] = __ldcg(theirs + (kTok + t) * kTileRows + rloc);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (g0 + i <= last) {
          v[0][t] += part[i][0];
          if (nacc == 2) v[1][t] += part[i][1];
        }
      }
    }
  }
  apply_epilogue(cx, ph, tile, rloc, v, t0, mt);
  return true;
}

// Projection phase on the tcgen05 engine, worker side.
__device__ bool worker_gemm_tc(const Ctx& cx, int gp, uint32_t& q, uint32_t& passed, int wtid) {
  const KParams& p = *cx.p;
  const GemmPhase* ph = p.phases + gp;
  const Range r = cta_range(ph, cx.cta, cx.grid);
  const int ntt = (p.m + kTok - 1) / kTok;
  const int tc = ph->tc, nacc = ph->nacc;
  const int quad = ((wtid >> 5) + 2) & 3;  // TMEM lane quadrant this warp may read
  const int rloc = quad * 32 + (wtid & 31);
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&cx.misc->tmem_base);
  for (int tt = 0; tt < ntt; ++tt) {
    // Partials and tile counters are reused by the next token tile.
    if (tt > 0 && !grid_barrier(cx, passed, wtid)) return false;
    if (r.c1 <= r.c0) continue;
    const int t0 = tt * kTok;
    const int mt = min(kTok, p.m - t0);
    trace_event(cx, wtid, EV_PHASE_ENTER);
    stage_b(cx, ph, r, t0, mt, wtid);
    trace_event(cx, wtid, EV_B_STAGED);
    long long c = r.c0;
    while (c < r.c1) {
      const int tile = static_cast<int>(c / tc);
      const long long tile_c0 = static_cast<long long>(tile) * tc;
      long long seg_end = tile_c0 + tc;
      if (seg_end > r.c1) seg_end = r.c1;
      const bool complete = (c == tile_c0) && (seg_end == tile_c0 + tc);
      const uint32_t buf = q & 1u;
      bool ok = wait_mbar(cx, smem_u32(&cx.misc->accfull[buf]), (q >> 1) & 1u, SITE_EPI_ACC, gp);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
      if (c == r.c0) trace_event(cx, wtid, EV_FIRST_ACC);
      tc_fence_after();
      float v[2][kTok];
      if (ok) {
        for (int a = 0; a < nacc; ++a) {
          const bool has = (nacc == 1) || (seg_end - c >= 2) || (((c & 1) != 0) == (a == 1));
          if (has) {
            tmem_ld16(tmem + (static_cast<uint32_t>(quad * 32) << 16) + (buf * 2u + a) * kTok, v[a]);
          } else {
#pragma unroll
            for (int t = 0; t < kTok; ++t) v[a][t] = 0.f;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&cx.misc->accempty[buf]));
      ++q;
      if (!workers_ok(cx, ok)) return false;
      if (complete) {
        apply_epilogue(cx, ph, tile, rloc, v, t0, mt);
      } else {
        if (!finish_split(cx, ph, r, tile, rloc, v, t0, mt, wtid)) return false;
      }
      c = seg_end;
    }
    trace_event(cx, wtid, EV_PHASE_DONE);
  }
  return true;
}

// Projection phase on the SIMT engine (bring-up / diagnostics): every worker
// warp of the grid takes output rows round-robin and does plain dot products.
__device__ __noinline__ bool worker_gemm_simt(const Ctx& cx, int gp, uint32_t& passed, int wtid) {
  const KParams& p = *cx.p;
  const GemmPhase* ph = p.phases + gp;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int k = ph->k;
  int tb = kBBytes / (k * 2);
  if (tb > kTok) tb = kTok;
  if (tb < 1) tb = 1;
  bf16* bs = reinterpret_cast<bf16*>(cx.smem_b);
  float v[2][kTok];
  for (int t0 = 0; t0 < p.m; t0 += tb) {
    const int mt = min(tb, p.m - t0);
    named_bar_sync(1, kWorkers);
    if (ph->bmode == B_NORM) norm_stats(cx, ph, t0, mt, wtid);
    for (int item = wtid; item < mt * (k / 8); item += kWorkers) {
      const int t = item / (k / 8), vec = item % (k / 8);
      const uint4 u = activation_vec(cx, ph, activation_row(p, ph, t0 + t), t, vec * 8);
      *reinterpret_cast<uint4*>(bs + t * k + vec * 8) = u;
    }
    named_bar_sync(1, kWorkers);
    const int total_rows = ph->ntiles * kTileRows;
    for (int row = cx.cta * kWorkerWarps + warp; row < total_rows; row += cx.grid * kWorkerWarps) {
      const int tile = row / kTileRows, rloc = row % kTileRows;
      for (int a = 0; a < ph->nacc; ++a) {
        const bf16* w;
        int n;
        if (ph->nacc == 2) {
          n = row;
          w = ph->w[a];
          if (n >= ph->n[0]) { for (int t = 0; t < mt; ++t) v[a][t] = 0.f; continue; }
        } else {
          const int seg = segment_of_tile(ph, tile);
          n = (tile - ph->tile_start[seg]) * kTileRows + rloc;
          w = ph->w[seg];
          if (n >= ph->n[seg]) { for (int t = 0; t < mt; ++t) v[a][t] = 0.f; continue; }
        }
        const uint4* wrow = reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * k);
        for (int t = 0; t < mt; ++t) v[a][t] = 0.f;
        for (int vec = lane; vec < k / 8; vec += 32) {
          float wf[8], xf[8];
          unpack8(__ldg(wrow + vec), wf);
          for (int t = 0; t < mt; ++t) {
            unpack8(*reinterpret_cast<const uint4*>(bs + t * k + vec * 8), xf);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[a][t] = fmaf(wf[e], xf[e], v[a][t]);
          }
        }
        for (int t = 0; t < mt; ++t) v[a][t] = warp_sum(v[a][t]);
      }
      if (lane == 0) apply_epilogue(cx, ph, tile, rloc, v, t0, mt);
    }
  }
  (void)passed;
  return true;
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
  int len;            // decode: filled positions before this call
  int decode;         // 1: append the new key/value at `len` and attend over [0, len]
  int rope;           // 1: rotate q and the new key while loading (decode)
  int causal;         // prefill without a mask tensor: key j <= query qi
  float scale;
};

// Publish one value per query head of this chunk, wait (bounded) until every
// chunk of the row group has published.
__device__ bool attn_exchange(const Ctx& cx, float* slots, uint32_t* counter, int rowg, int ch, int nch, int gs,
                              const float* mine, int wtid) {
  if (wtid < gs) __stcg(slots + (static_cast<size_t>(rowg) * kMaxChunks + ch) * 8 + wtid, mine[wtid]);
  __threadfence();
  named_bar_sync(1, kWorkers);
  if (wtid == 0) {
    red_release_add_u32(counter, 1u);
    uint32_t spins = 0;
    while (ld_relaxed_u32(counter) < static_cast<uint32_t>(nch)) {
      if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, rowg)) {
        cx.misc->wabort = 1;
        break;
      }
    }
    __threadfence();
  }
  named_bar_sync(1, kWorkers);
  return *reinterpret_cast<volatile int*>(&cx.misc->wabort) == 0;
}

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

__device__ __forceinline__ float ldcg_bf16(const bf16* ptr) {
  return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(ptr))));
}

// Softmax attention for every (sequence, kv head, query token) row group; all
// query heads of the kv head share one pass over K and V.  In decode the
// context is split into chunks across CTAs, which exchange the running max
// and sum through global memory so that every probability is rounded to bf16
// against the global normaliser, as the reference ops do:
//   decode  (kv_attention): score = bf16(q.k) * scale in fp32
//   prefill (attention):    score = bf16(bf16(q.k) * scale) (+ mask, rounded again)
// then fp32 softmax, probability rounded to bf16, fp32 value sum rounded once.
__device__ __noinline__ bool attention_phase(const Ctx& cx, const AttnArgs& A, int wtid) {
  const KParams& p = *cx.p;
  const int hd = p.head_dim, half = hd / 2;
  const int gs = p.q_heads / p.kv_heads;
  const int rows = p.batch * p.kv_heads * A.sq;
  const int n_max = A.decode ? A.len + 1 : A.klen;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int lpk = hd / 8;    // lanes per key (16 B each)
  const int kpw = 32 / lpk;  // keys per warp pass
  const int sub = lane / lpk, dg = lane % lpk;

  const int max_len = (kScoreBytes / 4 / gs) & ~7;
  int nch = 1;
  if (A.decode) {
    nch = cx.grid / rows;
    if (nch < 1) nch = 1;
    const int by_len = (n_max + 63) / 64;
    if (nch > by_len) nch = by_len;
    if (nch > kMaxChunks) nch = kMaxChunks;
    const int need = (n_max + max_len - 1) / max_len;
    if (nch < need) nch = need;
  }
  const int chunk = (n_max + nch - 1) / nch;
  const int units = rows * nch;

  float* sc = reinterpret_cast<float*>(cx.smem_b);                // [gs][chunk]
  float* qs = reinterpret_cast<float*>(cx.smem_b + kScoreBytes);  // [gs][hd]
  float* red = qs + 8 * 128;                                      // [4][128]
  bf16* kn = reinterpret_cast<bf16*>(red + 4 * 128);              // [hd]
  bf16* vn = kn + 128;                                            // [hd]
  float* stat = reinterpret_cast<float*>(vn + 128);               // [8]

  for (int u = cx.cta; u < units; u += cx.grid) {
    const int rowg = u / nch, ch = u - rowg * nch;
    const int bk = rowg / A.sq, qi = rowg - bk * A.sq;  // (sequence, kv head) index and query token
    const int b = bk / p.kv_heads, kvh = bk - b * p.kv_heads;
    const int n = A.decode ? n_max : (A.causal ? min(qi + 1, A.klen) : A.klen);
    const int j0 = ch * chunk;
    const int j1 = min(n, j0 + chunk);
    const int cl = max(0, j1 - j0);
    const int newpos = A.decode ? A.len : -1;
    const bool owner = A.decode && (A.len >= j0 && A.len < j1);
    named_bar_sync(1, kWorkers);  // previous unit is done with the scratch

    // --- load q (all heads of the group) and, in decode, the new key/value
    long long pos = 0;
    if (A.rope) {
      pos = p.pos[b];
      if (pos < 0 || pos >= p.max_positions) pos = 0;  // reported by the prologue
    }
    const int loads = A.decode ? gs + 1 : gs;
    for (int idx = wtid; idx < loads * half; idx += kWorkers) {
      const int g = idx / half, i = idx - g * half;
      const bf16* src = (g < gs) ? A.q + b * A.q_bstride + static_cast<long long>(qi) * A.q_ld + (kvh * gs + g) * hd
                                 : A.knew + static_cast<long long>(b) * A.new_ld + kvh * hd;
      float first = ldcg_bf16(src + i);
      float second = ldcg_bf16(src + i + half);
      if (A.rope) {
        const float c = ldg_bf16(p.cos_t + pos * hd + i);
        const float s = ldg_bf16(p.sin_t + pos * hd + i);
        rope_pair(first, second, c, s, p.rope_style, first, second);
      }
      if (g < gs) {
        qs[g * hd + i] = first;
        qs[g * hd + i + half] = second;
      } else {
        kn[i] = __float2bfloat16_rn(first);
        kn[i + half] = __float2bfloat16_rn(second);
      }
    }
    if (A.decode) {
      for (int i = wtid; i < hd; i += kWorkers)
        vn[i] = __float2bfloat16_rn(ldcg_bf16(A.vnew + static_cast<long long>(b) * A.new_ld + kvh * hd + i));
    }
    named_bar_sync(1, kWorkers);
    const bf16* kbase = A.k + b * A.kv_bstride + kvh * hd;
    const bf16* vbase = A.v + b * A.kv_bstride + kvh * hd;
    if (owner) {  // in-kernel KV append
      bf16* kd = A.k + b * A.kv_bstride + static_cast<long long>(A.len) * A.kv_ld + kvh * hd;
      bf16* vd = A.v + b * A.kv_bstride + static_cast<long long>(A.len) * A.kv_ld + kvh * hd;
      for (int i = wtid; i < hd; i += kWorkers) {
        kd[i] = kn[i];
        vd[i] = vn[i];
      }
    }
    const bf16* mrow = A.mask ? A.mask + (static_cast<long long>(b) * A.sq + qi) * A.klen : nullptr;

    // --- scores: eight keys per thread are loaded before any is used
    constexpr int kU = 8;
    const int pass = kWorkerWarps * kpw;
    for (int base = j0 + warp * kpw; base < j1; base += pass * kU) {
      uint4 ku[kU];
#pragma unroll
      for (int u8 = 0; u8 < kU; ++u8) {
        const int j = base + u8 * pass + sub;
        ku[u8] = make_uint4(0, 0, 0, 0);
        if (j < j1) {
          if (j == newpos) ku[u8] = *reinterpret_cast<const uint4*>(kn + dg * 8);
          else ku[u8] = __ldcg(reinterpret_cast<const uint4*>(kbase + static_cast<long long>(j) * A.kv_ld) + dg);
        }
      }
#pragma unroll
      for (int u8 = 0; u8 < kU; ++u8) {
        if (base + u8 * pass >= j1) break;  // warp-uniform
        const int j = base + u8 * pass + sub;
        float kf[8];
        unpack8(ku[u8], kf);
        for (int g = 0; g < gs; ++g) {
          const float* qv = qs + g * hd + dg * 8;
          float dot = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(qv[e], kf[e], dot);
          for (int o = 1; o < lpk; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          if (dg == 0 && j < j1) {
            float sv = bf16_round(dot) * A.scale;
            if (!A.decode) {
              sv = bf16_round(sv);
              if (mrow) sv = bf16_round(sv + ldg_bf16(mrow + j));
            }
            sc[g * chunk + (j - j0)] = sv;
          }
        }
      }
    }
    named_bar_sync(1, kWorkers);

    // --- max
    for (int g = 0; g < gs; ++g) {
      float m = -INFINITY;
      for (int i = wtid; i < cl; i += kWorkers) m = fmaxf(m, sc[g * chunk + i]);
      m = warp_max(m);
      if (lane == 0) red[warp * 8 + g] = m;
    }
    named_bar_sync(1, kWorkers);
    if (wtid < gs) stat[wtid] = fmaxf(fmaxf(red[wtid], red[8 + wtid]), fmaxf(red[16 + wtid], red[24 + wtid]));
    named_bar_sync(1, kWorkers);
    if (nch > 1) {
      if (!attn_exchange(cx, p.att_max, p.att_ctr + rowg * 4 + 0, rowg, ch, nch, gs, stat, wtid)) return false;
      if (wtid < gs) {
        float m = -INFINITY;
        for (int c = 0; c < nch; ++c)
          m = fmaxf(m, __ldcg(p.att_max + (static_cast<size_t>(rowg) * kMaxChunks + c) * 8 + wtid));
        stat[wtid] = m;
      }
      named_bar_sync(1, kWorkers);
    }

    // --- exp and sum
    for (int g = 0; g < gs; ++g) {
      const float m = stat[g];
      float s = 0.f;
      for (int i = wtid; i < cl; i += kWorkers) {
        const float e = expf(sc[g * chunk + i] - m);
        sc[g * chunk + i] = e;
        s += e;
      }
      s = warp_sum(s);
      if (lane == 0) red[32 + warp * 8 + g] = s;
    }
    named_bar_sync(1, kWorkers);
    if (wtid < gs) stat[wtid] = ((red[32 + wtid] + red[40 + wtid]) + red[48 + wtid]) + red[56 + wtid];
    named_bar_sync(1, kWorkers);
    if (nch > 1) {
      if (!attn_exchange(cx, p.att_sum, p.att_ctr + rowg * 4 + 1, rowg, ch, nch, gs, stat, wtid)) return false;
      if (wtid < gs) {
        float s = 0.f;
        for (int c = 0; c < nch; ++c) s += __ldcg(p.att_sum + (static_cast<size_t>(rowg) * kMaxChunks + c) * 8 + wtid);
        stat[wtid] = s;
      }
      named_bar_sync(1, kWorkers);
    }

    // --- probabilities (bf16) and value accumulation
    for (int g = 0; g < gs; ++g) {
      const float denom = stat[g];
      for (int i = wtid; i < cl; i += kWorkers) sc[g * chunk + i] = bf16_round(sc[g * chunk + i] / denom);
    }
    named_bar_sync(1, kWorkers);
    for (int g = 0; g < gs; ++g) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int base = j0 + warp * kpw; base < j1; base += pass * kU) {
        uint4 vu[kU];
#pragma unroll
        for (int u8 = 0; u8 < kU; ++u8) {
          const int j = base + u8 * pass + sub;
          vu[u8] = make_uint4(0, 0, 0, 0);
          if (j < j1) {
            if (j == newpos) vu[u8] = *reinterpret_cast<const uint4*>(vn + dg * 8);
            else vu[u8] = __ldcg(reinterpret_cast<const uint4*>(vbase + static_cast<long long>(j) * A.kv_ld) + dg);
          }
        }
#pragma unroll
        for (int u8 = 0; u8 < kU; ++u8) {
          const int j = base + u8 * pass + sub;
          if (j < j1) {
            float vf[8];
            unpack8(vu[u8], vf);
            const float pr = sc[g * chunk + (j - j0)];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(pr, vf[e], acc[e]);
          }
        }
      }
      for (int o = lpk; o < 32; o <<= 1) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
      }
      named_bar_sync(1, kWorkers);  // red is free (previous head consumed)
      if (sub == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) red[warp * 128 + dg * 8 + e] = acc[e];
      }
      named_bar_sync(1, kWorkers);
      if (wtid < hd) {
        const float o = ((red[wtid] + red[128 + wtid]) + red[256 + wtid]) + red[384 + wtid];
        const int head = kvh * gs + g;
        if (nch == 1) {
          A.out[b * A.out_bstride + static_cast<long long>(qi) * A.out_tstride + head * A.out_hstride + wtid] =
              __float2bfloat16_rn(o);
        } else {
          const size_t row = static_cast<size_t>(b) * p.q_heads + head;  // decode: sq == 1
          __stcg(p.att_part + (row * kMaxChunks + ch) * hd + wtid, o);
        }
      }
    }
    if (nch > 1) {
      __threadfence();
      named_bar_sync(1, kWorkers);
      if (wtid == 0) {
        const uint32_t old = atomicAdd(p.att_ctr + rowg * 4 + 2, 1u);
        const int is_last = (old == static_cast<uint32_t>(nch - 1));
        if (is_last) {  // every chunk is past both exchanges: safe to reset for the next use
          p.att_ctr[rowg * 4 + 0] = 0;
          p.att_ctr[rowg * 4 + 1] = 0;
          p.att_ctr[rowg * 4 + 2] = 0;
        }
        cx.misc->flag = is_last;
      }
      named_bar_sync(1, kWorkers);
      if (*reinterpret_cast<volatile int*>(&cx.misc->flag)) {
        __threadfence();
        for (int idx = wtid; idx < gs * hd; idx += kWorkers) {
          const int g = idx / hd, d = idx - g * hd;
          const int head = kvh * gs + g;
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

// Prefill: rotate q and k of every token in place in the qkv buffer.
__device__ __noinline__ void rope_phase(const Ctx& cx, int wtid) {
  const KParams& p = *cx.p;
  const int hd = p.head_dim, half = hd / 2;
  const int heads = p.q_heads + p.kv_heads;  // q heads then k heads are contiguous in a qkv row
  const long long items = static_cast<long long>(p.m) * heads * half;
  for (long long it = static_cast<long long>(cx.cta) * kWorkers + wtid; it < items;
       it += static_cast<long long>(cx.grid) * kWorkers) {
    const int i = static_cast<int>(it % half);
    const long long rest = it / half;
    const int h = static_cast<int>(rest % heads);
    const int t = static_cast<int>(rest / heads);
    long long pos = p.pos[t];
    if (pos < 0 || pos >= p.max_positions) pos = 0;
    bf16* x = p.qkv + static_cast<size_t>(t) * p.qkv_ld + h * hd;
    float first = ldcg_bf16(x + i), second = ldcg_bf16(x + i + half);
    const float c = ldg_bf16(p.cos_t + pos * hd + i);
    const float s = ldg_bf16(p.sin_t + pos * hd + i);
    rope_pair(first, second, c, s, p.prefill_rope_style, first, second);
    x[i] = __float2bfloat16_rn(first);
    x[i + half] = __float2bfloat16_rn(second);
  }
}

// ---------------------------------------------------------------------------
// workers: whole-launch schedule

__device__ void worker_loop(const Ctx& cx, int wtid) {
  const KParams& p = *cx.p;
  uint32_t q = 0, passed = 0;
  auto gemm = [&](int gp) -> bool {
    return p.engine == MK_ENGINE_SIMT ? worker_gemm_simt(cx, gp, passed, wtid) : worker_gemm_tc(cx, gp, q, passed, wtid);
  };
  const int q_size = p.q_heads * p.head_dim, kv_size = p.kv_heads * p.head_dim;
  AttnArgs A;
  A.knew = nullptr; A.vnew = nullptr; A.new_ld = 0; A.mask = nullptr;
  A.sq = 1; A.klen = 0; A.len = 0; A.decode = 0; A.rope = 0; A.causal = 0; A.scale = p.att_scale;
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
    A.len = *p.len[0]; A.decode = 1;
    if (!attention_phase(cx, A, wtid)) return;
    if (!grid_barrier(cx, passed, wtid)) return;
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
  // Layer 0's residual stream starts as the embedding rows.
  for (int v = cx.cta * kWorkers + wtid; v < p.m * (p.hidden / 8); v += cx.grid * kWorkers) {
    const int t = v / (p.hidden / 8), c = v - t * (p.hidden / 8);
    long long id = p.ids[t];
    if (id < 0 || id >= p.vocab) id = 0;
    reinterpret_cast<uint4*>(p.hidden_buf + static_cast<size_t>(t) * p.hidden)[c] =
        __ldg(reinterpret_cast<const uint4*>(p.embed + id * p.hidden) + c);
  }
  const bool decode = (p.mode == MODE_DECODE);
  int step = 0;
#define MK_DEBUG_STEP() do { if (p.debug_stop && ++step >= p.debug_stop) return; } while (0)
  MK_DEBUG_STEP();
  for (int layer = 0; layer < p.layers; ++layer) {
    if (!gemm(layer * 4 + 0)) return;                       // [RMSNorm] q, k, v (+bias)
    MK_DEBUG_STEP();
    if (!grid_barrier(cx, passed, wtid)) return;
    MK_DEBUG_STEP();
    A.q = p.qkv; A.q_ld = p.qkv_ld;
    A.out = p.attn; A.out_tstride = q_size; A.out_hstride = p.head_dim;
    if (decode) {
      A.q_bstride = p.qkv_ld;
      A.k = static_cast<bf16*>(p.kc[layer]); A.v = static_cast<bf16*>(p.vc[layer]);
      A.kv_bstride = static_cast<long long>(p.capacity) * kv_size; A.kv_ld = kv_size;
      A.knew = p.qkv + q_size; A.vnew = A.knew + kv_size; A.new_ld = p.qkv_ld;
      A.out_bstride = q_size;
      A.len = *p.len[layer]; A.decode = 1; A.rope = 1;
    } else {
      rope_phase(cx, wtid);
      if (!grid_barrier(cx, passed, wtid)) return;
      A.q_bstride = static_cast<long long>(p.seq) * p.qkv_ld;
      A.k = p.qkv + q_size; A.v = A.k + kv_size;
      A.kv_bstride = static_cast<long long>(p.seq) * p.qkv_ld; A.kv_ld = p.qkv_ld;
      A.out_bstride = static_cast<long long>(p.seq) * q_size;
      A.mask = p.mask; A.sq = p.seq; A.klen = p.seq; A.causal = (p.mask == nullptr);
    }
    if (!attention_phase(cx, A, wtid)) return;              // [RoPE] attention (+ KV append)
    trace_event(cx, wtid, EV_ATTENTION_DONE);
    MK_DEBUG_STEP();
    if (!grid_barrier(cx, passed, wtid)) return;
    if (decode && cx.cta == 0 && wtid == 0) *p.len[layer] = A.len + 1;  // publish after the interval closes
    MK_DEBUG_STEP();
    if (!gemm(layer * 4 + 1)) return;                       // o_proj + residual
    MK_DEBUG_STEP();
    if (!grid_barrier(cx, passed, wtid)) return;
    if (!gemm(layer * 4 + 2)) return;                       // [RMSNorm] gate, up -> SiLU*up
    MK_DEBUG_STEP();
    if (!grid_barrier(cx, passed, wtid)) return;
    if (!gemm(layer * 4 + 3)) return;                       // down + residual
    MK_DEBUG_STEP();
    if (!grid_barrier(cx, passed, wtid)) return;
  }
#undef MK_DEBUG_STEP
  gemm(p.layers * 4);                                       // [final RMSNorm] lm_head
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
  cx.smem_b = smem + kStages * kStageBytes;
  cx.misc = reinterpret_cast<SmemMisc*>(cx.smem_b + kBBytes);
  cx.deadline = clock64() + p.timeout_cycles;
  cx.cta = blockIdx.x;
  cx.grid = gridDim.x;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool tc = (p.engine == MK_ENGINE_TCGEN05) && p.n_gemm > 0;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&cx.misc->full[s]), 1);
      mbar_init(smem_u32(&cx.misc->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&cx.misc->accfull[b]), 1);
      mbar_init(smem_u32(&cx.misc->accempty[b]), kWorkers);
    }
    mbar_init(smem_u32(&cx.misc->bfull), kWorkers);
    cx.misc->wabort = 0;
    cx.misc->bad = 0;
    cx.misc->flag = 0;
    cx.misc->trace_n = 0;
    mbar_fence_init();
  }
  // Token rows a launch does not fill must not hold NaN patterns from earlier kernels.
  for (int i = tid; i < kBBytes / 16; i += kThreads) reinterpret_cast<uint4*>(cx.smem_b)[i] = make_uint4(0, 0, 0, 0);
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
        if (id < 0 || id >= p.vocab || pos < 0 || pos >= p.max_positions) bad = MK_STATUS_BAD_INDEX;
      }
    }
    if (p.mode != MODE_PREFILL) {
      const int nl = (p.mode == MODE_KVATT) ? 1 : p.layers;
      for (int l = tid; l < nl; l += kThreads) {
        const int len = *p.len[l];
        if (len < 0 || len + 1 > p.capacity) bad = MK_STATUS_KV_OVERFLOW;
      }
    }
    if (bad) atomicMax(&cx.misc->bad, bad);
  }
  __syncthreads();
  tc_fence_after();
  const int bad = *reinterpret_cast<volatile int*>(&cx.misc->bad);
  if (bad) {
    if (tid == 0) {
      if (cx.cta == 0 && atomicCAS(&cx.ctrl->status, 0, bad) == 0) {
        cx.ctrl->where = SITE_PROLOGUE;
        cx.ctrl->cta = 0;
        cx.ctrl->detail = 0;
      }
      // Keep the monotonic barrier counter consistent with what the host expects.
      if (p.nbar > 0) atomicAdd(&cx.ctrl->barrier, static_cast<uint32_t>(p.nbar));
    }
  } else if (warp == 0) {
    if (tc && tid == 0) producer_loop(cx);
  } else if (warp == 1) {
    if (tc && tid == 32) mma_loop(cx);
  } else {
    worker_loop(cx, tid - 64);
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
