// The decode megakernel for launches of at most four tokens (batch-1 decode is
// the case that matters).  Same phase tables, status protocol and bounded waits
// as mk::megakernel, but the weights are not consumed by tcgen05.
//
// Why not tcgen05 here: one tcgen05.mma of 128 weight rows by 16 token columns
// occupies the tensor pipe for ~78 cycles whatever the token count and however
// few of the 128 rows hold weights (an even split of a projection over 148 CTAs
// wants tiles of 14-56 rows), which capped a CTA at 6-12 bytes of weights per
// cycle where HBM can deliver 22.
//
// Roles: warp 0 = TMA producer (small_producer), warps 1-8 = consumers (operand
// staging with the RMSNorm fused in, projection, epilogue, decode attention).
// No TMEM, no MMA warp.  Two kernels are instantiated per token count:
//   <1, true>   the one-token row table: CUDA-core FMAs over plain weight rows
//               (small_gemm, small_gemm_rows), a single grid barrier per launch;
//   <T, false>  the split-K table for one to four tokens: warp-level mma.sync
//               over 128-byte-swizzled boxes (small_gemm_mma), two grid barriers
//               per layer.
//
// Weight copies are 14-34 KB each (a two- or three-dimensional tensor-map box,
// or whole contiguous rows through a 1-D bulk copy): an SM's copy engine retires
// about three copies per microsecond whatever their size.
//
// Phases hand their outputs over as 64-bit words {stamp, payload} that the
// consumer's staging polls (stamped_payloads): a reader that sees the stamp has
// the data, so no fence and no grid barrier is needed, and a consumer starts as
// soon as its own producers are done.
//
// Polls and barrier waits are compiler barriers for memory: whatever a loop
// needs from the context, the parameters or a descriptor is copied into locals
// before the loop (a kernel parameter read through the context is two dependent
// loads; one such read in a staging loop measured 40 us per step).
#pragma once
#include "decoder_kernel.cuh"

namespace mk {

constexpr int kSmallWarps = 8;
constexpr int kSmallWorkers = kSmallWarps * 32;
constexpr int kSmallThreads = 32 + kSmallWorkers;
constexpr int kXFloats = kBSlots * kChunkK;  // activation operand of one K slice per token, fp32 (one-token row table)
constexpr int kXElems = kBSlots * kChunkK;      // the same as bf16 for the mma.sync consumer (2048 elements)
constexpr int kXTokenBytes = kXElems * 2 + 16;  // its row pitch in shared memory (the padding spreads token rows over the banks)
// Weight ring of this kernel.  Measured on the 1.7B shape (batch 1, us per step): 92 KB with copies of
// up to 30 KB 1252; 120 KB / 36 KB 1185; 126 KB and more 1276-1310: past 196 KB of shared memory per CTA
// the carve-out jumps to 228 KB and the 28 KB of L1 that remain no longer hold the stack frames.
constexpr int kSmallRingGranules = 120;    // default; a handle may choose up to kSmallRingMax (KParams::small_ring)
constexpr int kSmallRingMax = 152;
constexpr int small_smem_bytes(int ring_granules) { return 1024 + ring_granules * kGranule + kBBytes + kMiscBytes; }
static_assert(small_smem_bytes(kSmallRingMax) <= 232448, "the largest ring exceeds 227 KiB of shared memory");
static_assert(kSplitTokens * kXFloats * 4 <= kBBytes, "activation operand does not fit its region");

struct SmallState {
  int head, seq;    // weight ring replay, the producer's sequence
  uint32_t passed;  // grid barriers passed
};

__device__ __forceinline__ void small_sync() { named_bar_sync(1, kSmallWorkers); }

__device__ __forceinline__ bool small_ok(const Ctx& cx, bool ok) {
  if (!ok) cx.misc->wabort = 1;
  small_sync();
  return *reinterpret_cast<volatile int*>(&cx.misc->wabort) == 0;
}

// Grid barrier in two halves so that loads which do not depend on other CTAs
// can be issued between the arrival and the wait.
__device__ __forceinline__ void small_arrive(const Ctx& cx, SmallState& st, int wtid) {
  small_sync();  // every consumer's stores are done (bar.sync orders them before thread 0's release)
  st.passed += 1;
  if (wtid == 0) red_release_add_u32(&cx.ctrl->barrier, 1u);
}

__device__ __forceinline__ bool small_wait(const Ctx& cx, SmallState& st, int wtid) {
  if (wtid == 0) {
    const uint32_t target = cx.misc->epoch + st.passed * static_cast<uint32_t>(cx.grid);
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_relaxed_u32(&cx.ctrl->barrier) - target) < 0) {
      if ((++spins & 255u) == 0 && give_up(cx, SITE_GRID_BARRIER, static_cast<int>(st.passed))) {
        cx.misc->wabort = 1;
        break;
      }
    }
    __threadfence();
  }
  small_sync();
  trace_event(cx, wtid, EV_BARRIER_DONE);
  return *reinterpret_cast<volatile int*>(&cx.misc->wabort) == 0;
}

// The next phase's descriptor: requested when a phase starts, put into shared memory when the
// phase has finished (a warp stalls on the store until its load has returned).
__device__ __forceinline__ uint32_t small_phase_word(const Ctx& cx, int gp, int wtid) {
  if (gp >= cx.misc->n_gemm || wtid >= static_cast<int>(sizeof(GemmPhase) / 4)) return 0u;
  return __ldg(reinterpret_cast<const uint32_t*>(cx.misc->phases + gp) + wtid);
}
__device__ __forceinline__ void small_phase_store(const Ctx& cx, int gp, int wtid, uint32_t word) {
  if (gp >= cx.misc->n_gemm || wtid >= static_cast<int>(sizeof(GemmPhase) / 4)) return;
  reinterpret_cast<uint32_t*>(&cx.misc->phase[gp & 1])[wtid] = word;
}
static_assert(sizeof(GemmPhase) / 4 <= kSmallWorkers, "one word of the phase descriptor per consumer thread");

// Wait (bounded) until a 64-bit word carries `stamp` in its upper half; the lower half is the payload.
__device__ __forceinline__ uint32_t stamped_payload(const Ctx& cx, const unsigned long long* word, uint32_t stamp, bool& fresh) {
  unsigned long long w = ld_relaxed_u64(word);
  uint32_t spins = 0;
  while (static_cast<uint32_t>(w >> 32) != stamp) {
    if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, -1)) {
      fresh = false;
      break;
    }
    w = ld_relaxed_u64(word);
  }
  return static_cast<uint32_t>(w);
}

// The same for N consecutive words (N even, 16-byte aligned): every load is issued before any stamp
// is looked at, and only a stale batch is read again.
template <int N>
__device__ __forceinline__ void stamped_payloads(const Ctx& cx, const unsigned long long* words, uint32_t stamp, bool& fresh,
                                                 uint32_t* out) {
  uint32_t spins = 0;
  while (true) {
    unsigned long long w[N];
#pragma unroll
    for (int i = 0; i < N; i += 2) ld_relaxed_v2_u64(words + i, w[i], w[i + 1]);
    bool all = true;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      all = all && static_cast<uint32_t>(w[i] >> 32) == stamp;
      out[i] = static_cast<uint32_t>(w[i]);
    }
    if (all) return;
    __nanosleep(32);  // hundreds of CTAs poll the same lines: leave the L2 to the producers' stores (32 / 128 / 512 ns: 1 106 / 1 109 / 1 116 us per step)
    if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, -1)) {
      fresh = false;
      return;
    }
  }
}

// fp32 operand layout: per token kXFloats floats; inside a 64-element K chunk the
// eight 8-element vectors are stored as two float4 halves, 128 bytes apart, so
// that the eight lanes sharing a weight row read 128 contiguous bytes per load.
__device__ __forceinline__ float* x_slot(uint8_t* region, int t, int chunk, int vec) {
  return reinterpret_cast<float*>(region) + t * kXFloats + chunk * kChunkK + vec * 4;
}
template <bool ROW>
__device__ __forceinline__ void x_store(uint8_t* region, int t, int chunk, int vec, const float* f) {
  if constexpr (ROW) {  // one-token row table: fp32 for the CUDA-core consumer
    float* dst = x_slot(region, t, chunk, vec);
    *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + 32) = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    // mma.sync consumer: bf16 (exact: every operand is a bf16 tensor in the reference), one row of K elements per token
    *reinterpret_cast<uint4*>(region + t * kXTokenBytes + (chunk * kChunkK + vec * 8) * 2) = pack8(f);
  }
}

// RMSNorm fused with staging (K = hidden <= 2048: one 8-element vector per
// thread and token).  Also applies the pending residual update of the split-K
// table: x = residual + bf16(sum of the previous projection's fp32 K-slice
// partials, in slice order), writes this CTA's share of x back as the new
// residual stream, and normalises x with the two roundings of the Hugging Face
// RMSNorm.  `wu` is this thread's vector of the norm weight, loaded by the
// caller before the grid barrier opened.
template <bool ROW>
__device__ __noinline__ bool small_stage_norm(const Ctx& cx, const GemmPhase* ph, int mt, int wtid, uint4 wu, uint32_t stamp) {
  const KParams& p = *cx.p;
  const int warp = wtid >> 5, lane = wtid & 31;
  // Everything the token loop needs, read once: the polls below are compiler barriers for memory, and the
  // context, the parameters and the descriptor would otherwise be read again behind each of them.
  const int k = ph->k, nvec = k / 8;
  const int parts = ph->add_parts;
  const int writers = min(cx.grid, ph->nunits);
  const int cta = cx.cta, m = p.m;
  const float eps = p.eps;
  const unsigned long long* ll_src = ph->ll_src;
  const int ll_src_ld = ph->ll_src_ld;
  const float* partial = ph->partial;
  bf16* h_out = ph->h_out;
  uint8_t* region = cx.smem_b;
  float (*sred)[8] = cx.misc->sred;
  const bool active = wtid < nvec;
  bool fresh = true;
  float w[8];
  unpack8(wu, w);
  for (int t = 0; t < mt; ++t) {
    float f[8];
    uint4 xu = make_uint4(0, 0, 0, 0);
    if (active && ll_src != nullptr) {
      // the residual stream as stamped bf16 pairs (one-token row table): waiting for the stamps of the
      // previous projection's epilogues replaces the grid barrier; nothing is added, nothing written back
      uint32_t pair[4];
      stamped_payloads<4>(cx, ll_src + static_cast<size_t>(t) * ll_src_ld + wtid * 4, stamp, fresh, pair);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(pair[i] << 16);
        f[2 * i + 1] = __uint_as_float(pair[i] & 0xFFFF0000u);
      }
    } else if (active) {
      const uint4* row = reinterpret_cast<const uint4*>(activation_row(p, ph, t));
      xu = __ldcg(row + wtid);
      float4 lo[kMaxSplit], hi[kMaxSplit];
#pragma unroll
      for (int s8 = 0; s8 < kMaxSplit; ++s8) {
        if (s8 < parts) {
          const float4* part = reinterpret_cast<const float4*>(partial + (static_cast<size_t>(s8) * m + t) * k) + wtid * 2;
          lo[s8] = __ldcg(part);
          hi[s8] = __ldcg(part + 1);
        }
      }
      unpack8(xu, f);
      if (parts > 0) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s8 = 0; s8 < kMaxSplit; ++s8) {
          if (s8 < parts) {
            acc[0] += lo[s8].x; acc[1] += lo[s8].y; acc[2] += lo[s8].z; acc[3] += lo[s8].w;
            acc[4] += hi[s8].x; acc[5] += hi[s8].y; acc[6] += hi[s8].z; acc[7] += hi[s8].w;
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = bf16_round(f[e] + bf16_round(acc[e]));
        xu = pack8(f);
      }
      if (h_out && (wtid * writers) / nvec == cta)
        __stcg(reinterpret_cast<uint4*>(h_out + static_cast<size_t>(t) * k) + wtid, xu);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) sum = fmaf(f[e], f[e], sum);
    sum = warp_sum(sum);
    if (lane == 0) sred[t][warp] = sum;
    small_sync();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kSmallWarps; ++i) total += sred[t][i];
    const float r = 1.0f / sqrtf(total / static_cast<float>(k) + eps);
    if (active) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = bf16_round(w[e] * bf16_round(f[e] * r));
      x_store<ROW>(region, t, wtid >> 3, wtid & 7, f);
    }
  }
  return fresh;
}

// Plain or attention-output operand: K chunks [k0, k0 + count) of every token.  One vector per
// thread and trip (256 vectors cover a 2048-element slice of one token); kept small on purpose.
template <bool ROW>
__device__ __noinline__ bool small_stage_cols(const Ctx& cx, const GemmPhase* ph, int k0, int count, int mt, int wtid,
                                              int nch, uint32_t stamp) {
  const KParams& p = *cx.p;
  // read once: every poll below is a compiler barrier for memory
  const unsigned long long* ll_src = ph->ll_src;
  const int ll_src_ld = ph->ll_src_ld, bmode = ph->bmode;
  const int head_dim = p.head_dim, q_heads = p.q_heads;
  uint8_t* region = cx.smem_b;
  const int per_token = count * 8;
  const int items = per_token * mt;
  bool fresh = true;
#pragma unroll 1
  for (int item = wtid; item < items; item += kSmallWorkers) {
    const int t = item / per_token, rem = item - t * per_token;
    const int col = (k0 + (rem >> 3)) * kChunkK + (rem & 7) * 8;
    float f[8];
    if (ll_src != nullptr && bmode == B_PLAIN) {
      // stamped bf16 pairs written by the producing phase's epilogues: waiting for the stamps is the synchronisation
      const unsigned long long* words = ll_src + static_cast<size_t>(t) * ll_src_ld + (col >> 1);
      uint32_t pair[4];
      stamped_payloads<4>(cx, words, stamp, fresh, pair);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(pair[i] << 16);
        f[2 * i + 1] = __uint_as_float(pair[i] & 0xFFFF0000u);
      }
    } else if (ll_src != nullptr) {
      // stamped fp32 chunk partials of the attention phase, summed in chunk order and rounded once
      const int head = col / head_dim, d = col - head * head_dim;
      const unsigned long long* part = ll_src + (static_cast<size_t>(t) * q_heads + head) * kMaxChunks * head_dim + d;
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
#pragma unroll 1
      for (int c = 0; c < nch; ++c) {
        uint32_t bits[8];
        stamped_payloads<8>(cx, part + c * head_dim, stamp, fresh, bits);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += __uint_as_float(bits[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = bf16_round(f[e]);
    } else {
      const uint4 u = (bmode == B_ATTN) ? attention_vec(p, t, col, nch)
                                            : __ldcg(reinterpret_cast<const uint4*>(activation_row(p, ph, t) + col));
      unpack8(u, f);
    }
    x_store<ROW>(region, t, rem >> 3, rem & 7, f);
  }
  return fresh;
}

// Row sums of one unit wait in shared memory ([accumulator][row][token]) between the K loop and
// the epilogue, which thread r runs for row r.
constexpr int kRowSumOffset = kSplitTokens * kXFloats * 4;  // behind the activation operand
constexpr int kSmallTileRows = 64;                          // tile height of the small-launch table
static_assert(kRowSumOffset + 2 * kSmallTileRows * kSplitTokens * 4 <= kBBytes, "row sums do not fit");

// Cross-warp partial sums of the mma.sync consumer: [warp][accumulator][row][token], behind its bf16 operand.
constexpr int kPartOffset = 20 * 1024;
constexpr int kPartFloats = kSmallWarps * 2 * kSmallTileRows * kSplitTokens;
static_assert(kSplitTokens * kXTokenBytes <= kPartOffset, "activation operand overlaps the partial sums");
static_assert(kPartOffset + kPartFloats * 4 <= kBBytes, "partial sums do not fit");

// Sum of the eight warps' partials of (accumulator a, row r, token t), in warp order.
__device__ __forceinline__ float small_row_sum(const float* part, int a, int r, int t) {
  float v = 0.f;
#pragma unroll
  for (int w8 = 0; w8 < kSmallWarps; ++w8) v += part[((w8 * 2 + a) * kSmallTileRows + r) * kSplitTokens + t];
  return v;
}

template <int T, bool ROW>
__device__ __noinline__ void small_finish_row(const Ctx& cx, const GemmPhase* ph, int seg, int slice, int n, int r,
                                              uint32_t* bits) {
  float v[2][T];
  if constexpr (ROW) {
    const float* sums = reinterpret_cast<const float*>(cx.smem_b + kRowSumOffset);
#pragma unroll
    for (int t = 0; t < T; ++t) {
      v[0][t] = sums[r * kSplitTokens + t];
      v[1][t] = sums[(kSmallTileRows + r) * kSplitTokens + t];
    }
  } else {
    const float* part = reinterpret_cast<const float*>(cx.smem_b + kPartOffset);
#pragma unroll
    for (int t = 0; t < T; ++t) {
      v[0][t] = small_row_sum(part, 0, r, t);
      v[1][t] = ph->nacc == 2 ? small_row_sum(part, 1, r, t) : 0.f;
    }
  }
  if (ph->ll) {  // the caller sends the rounded outputs as stamped words
    if (ph->epi == EPI_ROWRES) {  // new residual = residual + bf16(projection)
#pragma unroll
      for (int t = 0; t < T; ++t) {
        float old;
        if (ph->gather) {
          old = ldg_bf16(activation_row(*cx.p, ph, t) + n);
        } else {
          const uint32_t pair = static_cast<uint32_t>(ld_relaxed_u64(ph->res_src + static_cast<size_t>(t) * ph->ll_ld + (n >> 1)));
          old = __uint_as_float((n & 1) ? (pair & 0xFFFF0000u) : (pair << 16));
        }
        bits[t] = __bfloat16_as_ushort(__float2bfloat16_rn(old + bf16_round(v[0][t])));
      }
    } else if (ph->epi == EPI_SILU) {
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const float act = bf16_round(silu(bf16_round(v[0][t])));
        bits[t] = __bfloat16_as_ushort(__float2bfloat16_rn(act * bf16_round(v[1][t])));
      }
    } else {
      const float bias = ph->bias[seg] ? ldg_bf16(ph->bias[seg] + n) : 0.f;
#pragma unroll
      for (int t = 0; t < T; ++t) bits[t] = __bfloat16_as_ushort(__float2bfloat16_rn(v[0][t] + bias));
    }
    return;
  }
  if (ph->epi == EPI_PARTIAL) {
    store_partial<T>(cx, ph, slice, n, v[0], 0, T);
  } else {
    float pre[T];
    pre[0] = (ph->epi == EPI_STORE && ph->bias[seg]) ? ldg_bf16(ph->bias[seg] + n) : 0.f;
    if (ph->epi == EPI_RESIDUAL) epilogue_prefetch<T>(cx, ph, seg, n, 0, T, pre);
    apply_epilogue<T>(cx, ph, seg, n, v, pre, 0, T);
  }
}

// Projection phase gp for this CTA's units.  The caller has made the phase descriptor visible in
// cx.misc->phase[gp & 1]; `wu` is the norm-weight vector for B_NORM phases.
//
// A weight copy holds [rows][kb * 64] bf16, plain rows.  The lanes of a warp split the K range of
// the copy: lane l keeps its eight activation values (per token) in registers for the whole copy
// and reads its 16 bytes of one row with one shared load; the warp walks the rows w, w + 8, ...
// (two or four rows at once when a row segment is shorter than 512 bytes).  Every (row, lane)
// keeps one fp32 chain over the K loop; at the end a fixed shuffle tree adds the lanes of a row.
// Accumulation order depends only on the CTA's rotated chunk order: no dependence on timing.
template <int N>
struct IntTag {
  static constexpr int value = N;
};

// One weight copy's share of a lane: ITERS rows, 4096 bytes apart, eight weights of each.  All loads
// first, then one FMA chain per row (the chains are independent, so they overlap).  Rows past the
// tile's last row read whatever the ring holds there; their sums are never stored.
template <int T, int ITERS>
__device__ __forceinline__ void small_fma_rows(uint32_t base, const float (&xf)[T][8], float (&acc)[8][T]) {
  uint4 w[ITERS];
#pragma unroll
  for (int i = 0; i < ITERS; ++i) w[i] = lds_v4(base + i * 4096);
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    float wf[8];
    unpack8(w[i], wf);
#pragma unroll
    for (int t = 0; t < T; ++t)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][t] = fmaf(wf[e], xf[t][e], acc[i][t]);
  }
}

template <int T, int NACC>
__device__ __noinline__ bool small_gemm(const Ctx& cx, int gp, SmallState& st, int wtid, uint4 wu, int nch, uint32_t stamp) {
  const GemmPhase* ph = &cx.misc->phase[gp & 1];
  const int nunits = ph->nunits, rows = ph->rows, ksplit = ph->ksplit, kslice = ph->kslice, gran = ph->gran;
  const bool per_unit = ksplit > 1;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int kb = ph->kb;                          // 1, 2 or 4 K chunks per copy
  const int lpr = kb * 8;                         // lanes per row
  const int rset = 32 / lpr;                      // rows a warp reads at once
  const int sel = lane / lpr, cl = lane - sel * lpr;
  const int row_first = warp * rset + sel;        // this lane's rows: row_first + i * 8 * rset
  const int iters = (rows + 8 * rset - 1) / (8 * rset);  // <= 8
  const uint32_t row_bytes = static_cast<uint32_t>(kb) * 128u;
  const uint32_t lane_off = row_first * row_bytes + (cl << 4);
  const int rot = k_rotation(cx.cta, cx.grid, kslice / kb) * kb;
  const uint32_t ring_base = smem_u32(cx.smem_a);
  const int ring_granules = cx.p->small_ring;
  const uint32_t x_base = smem_u32(cx.smem_b) + ((cl >> 3) * kChunkK + (cl & 7) * 4) * 4;
  float* sums = reinterpret_cast<float*>(cx.smem_b + kRowSumOffset);
  // barrier addresses and loop bounds in registers: the waits below are compiler barriers for memory
  const uint32_t full0 = smem_u32(&cx.misc->full[0]), empty0 = smem_u32(&cx.misc->empty[0]);
  const int my_cta = cx.cta, grid = cx.grid;
  const bool tracing = wtid == 0 && cx.misc->trace_on != 0;
  int head = st.head, seq = st.seq;
  bool ok = true;
  if (my_cta < nunits) {
    if (tracing) trace_event(cx, wtid, EV_PHASE_ENTER);
#pragma unroll 1
    for (int unit = my_cta; unit < nunits; unit += grid) {
      const int tile = unit / ksplit, slice = unit - tile * ksplit;
      if (per_unit || unit == my_cta) {
        if (unit != my_cta) small_sync();  // the previous unit has finished reading the operand
        // a normalising phase that opens a layer (or the lm_head) reads what the previous layer stamped
        if (ph->bmode == B_NORM) ok = small_stage_norm<true>(cx, ph, T, wtid, wu, (gp & 3) == 0 ? stamp - 1u : stamp) && ok;
        else ok = small_stage_cols<true>(cx, ph, slice * kslice, kslice, T, wtid, nch, stamp) && ok;
        small_sync();
        if (tracing && unit == my_cta) trace_event(cx, wtid, EV_B_STAGED);
      }
      int seg, row0;
      tile_origin(ph, tile, seg, row0);
      float acc[NACC][8][T];
#pragma unroll
      for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int t = 0; t < T; ++t) acc[a][i][t] = 0.f;
      int slot = rot;
      // The K loop, instantiated once per row-iteration count for one-token launches (ITERS > 0: no
      // predicate inside the unrolled body, so the loads of a copy issue back to back and the rows' FMA
      // chains interleave), and once in the general, predicated form (ITERS == 0).
      auto k_loop = [&](auto iters_tag) {
      constexpr int ITERS = decltype(iters_tag)::value;
#pragma unroll 1
      for (int k0 = 0; k0 < kslice; k0 += kb) {
        // this lane's activation values for the K range of the copy
        float xf[T][8];
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const uint4 lo = lds_v4(x_base + (t * kXFloats + slot * kChunkK) * 4);
          const uint4 hi = lds_v4(x_base + (t * kXFloats + slot * kChunkK + 32) * 4);
          xf[t][0] = __uint_as_float(lo.x); xf[t][1] = __uint_as_float(lo.y);
          xf[t][2] = __uint_as_float(lo.z); xf[t][3] = __uint_as_float(lo.w);
          xf[t][4] = __uint_as_float(hi.x); xf[t][5] = __uint_as_float(hi.y);
          xf[t][6] = __uint_as_float(hi.z); xf[t][7] = __uint_as_float(hi.w);
        }
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
          if (head + gran > ring_granules) head = 0;
          const uint32_t base = ring_base + head * kGranule + lane_off;
          head += gran;
          const uint32_t bar = seq % kChunkBars;
          // After a failed wait the warp keeps walking the schedule without waiting, so that
          // every consumer still reaches the same block-wide barriers and leaves together.
          const bool got = ok && wait_mbar(cx, full0 + bar * 8u, (seq / kChunkBars) & 1, SITE_MMA_FULL, gp);
          ok = __all_sync(0xffffffffu, got);
          if (tracing && k0 == 0 && a == 0 && unit == my_cta) trace_event(cx, wtid, EV_FIRST_COPY);
          if constexpr (ITERS > 0) {
            small_fma_rows<T, ITERS>(base, xf, acc[a]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (i < iters && row_first + i * 8 * rset < rows) {
                float wf[8];
                unpack8(lds_v4(base + i * 4096), wf);  // 8 * rset rows of row_bytes = 4096 bytes further on
#pragma unroll
                for (int t = 0; t < T; ++t)
#pragma unroll
                  for (int e = 0; e < 8; ++e) acc[a][i][t] = fmaf(wf[e], xf[t][e], acc[a][i][t]);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + bar * 8u);
          seq += 1;
        }
        slot = (slot + kb == kslice) ? 0 : slot + kb;
      }
      };
      if constexpr (T == 1) {
        switch (iters) {
          case 1: k_loop(IntTag<1>{}); break;
          case 2: k_loop(IntTag<2>{}); break;
          case 3: k_loop(IntTag<3>{}); break;
          case 4: k_loop(IntTag<4>{}); break;
          case 5: k_loop(IntTag<5>{}); break;
          case 6: k_loop(IntTag<6>{}); break;
          case 7: k_loop(IntTag<7>{}); break;
          default: k_loop(IntTag<8>{}); break;
        }
      } else {
        k_loop(IntTag<0>{});
      }
      if (tracing && unit == my_cta) trace_event(cx, wtid, EV_FIRST_ACC);
      if (unit != my_cta) small_sync();  // the previous unit's rows have been finished: `sums` is free
      if (lpr == 32) {
        // A row spans the warp: halve the rows a lane carries at each exchange (16, 8, 4), then add
        // the last four lanes; 9 shuffles for eight rows instead of 40.  Lane l with (l & 3) == 0
        // ends with row index i = bits 4, 3, 2 of l.
#pragma unroll
        for (int a = 0; a < NACC; ++a)
#pragma unroll
          for (int t = 0; t < T; ++t) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = acc[a][i][t];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const bool up = lane & 16;
              const float send = up ? v[i] : v[i + 4], keep = up ? v[i + 4] : v[i];
              v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const bool up = lane & 8;
              const float send = up ? v[i] : v[i + 2], keep = up ? v[i + 2] : v[i];
              v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
            }
            {
              const bool up = lane & 4;
              const float send = up ? v[0] : v[1], keep = up ? v[1] : v[0];
              v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
            }
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
            const int i = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
            const int r = warp + i * 8;
            if ((lane & 3) == 0 && r < rows) sums[(a * kSmallTileRows + r) * kSplitTokens + t] = v[0];
          }
      } else {
#pragma unroll 1
        for (int i = 0; i < iters; ++i) {
#pragma unroll
          for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int t = 0; t < T; ++t) {
              float x = 0.f;
#pragma unroll
              for (int i2 = 0; i2 < 8; ++i2) x = (i2 == i) ? acc[a][i2][t] : x;
              x += __shfl_xor_sync(0xffffffffu, x, 1);
              x += __shfl_xor_sync(0xffffffffu, x, 2);
              x += __shfl_xor_sync(0xffffffffu, x, 4);
              if (lpr > 8) x += __shfl_xor_sync(0xffffffffu, x, 8);
              const int r = row_first + i * 8 * rset;
              if (cl == 0 && r < rows) sums[(a * kSmallTileRows + r) * kSplitTokens + t] = x;
            }
        }
      }
      small_sync();
      {
        const bool mine = wtid < rows && row0 + wtid < ph->n[seg];
        uint32_t bits[T];
#pragma unroll
        for (int t = 0; t < T; ++t) bits[t] = 0u;
        if (mine) small_finish_row<T, true>(cx, ph, seg, slice, row0 + wtid, wtid, bits);
        if (ph->ll) {
          // Rows 2k and 2k + 1 (even tile height, even segment sizes) share a word:
          // {stamp, bf16 of the odd column, bf16 of the even column}, one 64-bit store.
          const int col = ph->out_col[seg] + row0 + wtid;
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const uint32_t other = __shfl_xor_sync(0xffffffffu, bits[t], 1);
            if (mine && !(wtid & 1))
              st_relaxed_u64(ph->ll_dst + static_cast<size_t>(t) * ph->ll_ld + (col >> 1),
                             (static_cast<unsigned long long>(stamp) << 32) | (other << 16) | bits[t]);
          }
        }
      }
    }
    if (tracing) trace_event(cx, wtid, EV_PHASE_DONE);
  }
  st.head = head;
  st.seq = seq;
  return ok;
}

// One-token projection whose tile is `rows` whole weight rows fetched as contiguous bytes (o_proj and
// down_proj of the row table).  The 256 consumer threads split a row: thread t owns the 8-element
// vectors t, t + 256, ... of every row and keeps its activation values in registers for the whole
// tile; a copy brings 1-8 rows; per row one fp32 chain per thread, a warp shuffle tree, and the
// eight warp sums are added in warp order by the thread that finishes the row.
__device__ __noinline__ bool small_gemm_rows(const Ctx& cx, int gp, SmallState& st, int wtid, int nch, uint32_t stamp) {
  const GemmPhase* ph = &cx.misc->phase[gp & 1];
  const int nunits = ph->nunits, rows = ph->rows, gran = ph->gran, rpc = ph->rpc, kc = ph->kc;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int kvecs = ph->k / 8;
  const uint32_t ring_base = smem_u32(cx.smem_a);
  const int ring_granules = cx.p->small_ring;
  const uint32_t row_bytes = static_cast<uint32_t>(ph->k) * 2u;
  float* sums = reinterpret_cast<float*>(cx.smem_b + kRowSumOffset);   // [row][warp] here
  // barrier addresses and loop bounds in registers: the waits below are compiler barriers for memory
  const uint32_t full0 = smem_u32(&cx.misc->full[0]), empty0 = smem_u32(&cx.misc->empty[0]);
  const int my_cta = cx.cta, grid = cx.grid;
  const bool tracing = wtid == 0 && cx.misc->trace_on != 0;
  const float* const xsrc = reinterpret_cast<const float*>(cx.smem_b);
  int head = st.head, seq = st.seq;
  bool ok = true;
  if (my_cta < nunits) {
    if (tracing) trace_event(cx, wtid, EV_PHASE_ENTER);
#pragma unroll 1
    for (int unit = my_cta; unit < nunits; unit += grid) {
      if (unit != my_cta) small_sync();
      ok = small_stage_cols<true>(cx, ph, 0, kc, 1, wtid, nch, stamp) && ok;
      small_sync();
      if (tracing && unit == my_cta) trace_event(cx, wtid, EV_B_STAGED);
      const int row0 = unit * rows;
      const int tile_rows = min(rows, ph->n[0] - row0);
      float xr[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = wtid + j * kSmallWorkers;
        if (v < kvecs) {
          const float* src = xsrc + (v >> 3) * kChunkK + (v & 7) * 4;
          const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 32);
          xr[j][0] = lo.x; xr[j][1] = lo.y; xr[j][2] = lo.z; xr[j][3] = lo.w;
          xr[j][4] = hi.x; xr[j][5] = hi.y; xr[j][6] = hi.z; xr[j][7] = hi.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) xr[j][e] = 0.f;
        }
      }
#pragma unroll 1
      for (int r0 = 0; r0 < tile_rows; r0 += rpc) {
        if (head + gran > ring_granules) head = 0;
        const uint32_t base = ring_base + head * kGranule + (wtid << 4);
        head += gran;
        const uint32_t bar = seq % kChunkBars;
        const bool got = ok && wait_mbar(cx, full0 + bar * 8u, (seq / kChunkBars) & 1, SITE_MMA_FULL, gp);
        ok = __all_sync(0xffffffffu, got);
        if (tracing && r0 == 0 && unit == my_cta) trace_event(cx, wtid, EV_FIRST_COPY);
        const int count = min(rpc, tile_rows - r0);
        // G rows of the copy at a time: their loads issue together and their FMA chains and shuffle
        // trees interleave (one row alone is a chain of up to 32 dependent FMAs and 5 dependent shuffles).
        // A group that runs past the copy repeats its last row and drops the repeats.
        auto row_groups = [&](auto group_tag) {
          constexpr int G = decltype(group_tag)::value;
#pragma unroll 1
          for (int r = 0; r < count; r += G) {
            float acc[G];
            uint32_t at[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
              acc[g] = 0.f;
              at[g] = base + static_cast<uint32_t>(min(r + g, count - 1)) * row_bytes;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (wtid + j * kSmallWorkers < kvecs) {
                uint4 w[G];
#pragma unroll
                for (int g = 0; g < G; ++g) w[g] = lds_v4(at[g] + j * (kSmallWorkers * 16));
#pragma unroll
                for (int g = 0; g < G; ++g) {
                  float wf[8];
                  unpack8(w[g], wf);
#pragma unroll
                  for (int e = 0; e < 8; ++e) acc[g] = fmaf(wf[e], xr[j][e], acc[g]);
                }
              }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
              for (int g = 0; g < G; ++g) acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], o);
            if (lane == 0) {
#pragma unroll
              for (int g = 0; g < G; ++g)
                if (r + g < count) sums[(r0 + r + g) * kSmallWarps + warp] = acc[g];
            }
          }
        };
        if (rpc >= 4) row_groups(IntTag<4>{});
        else if (rpc >= 2) row_groups(IntTag<2>{});
        else row_groups(IntTag<1>{});
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + bar * 8u);
        seq += 1;
      }
      if (tracing && unit == my_cta) trace_event(cx, wtid, EV_FIRST_ACC);
      small_sync();
      {
        const bool mine = wtid < tile_rows;
        uint32_t bits = 0u;
        if (mine) {
          float y = sums[wtid * kSmallWarps];
#pragma unroll
          for (int w8 = 1; w8 < kSmallWarps; ++w8) y += sums[wtid * kSmallWarps + w8];
          const int n = row0 + wtid;
          float old;
          if (ph->gather) {
            old = ldg_bf16(activation_row(*cx.p, ph, 0) + n);
          } else {
            const uint32_t pair = static_cast<uint32_t>(ld_relaxed_u64(ph->res_src + (n >> 1)));
            old = __uint_as_float((n & 1) ? (pair & 0xFFFF0000u) : (pair << 16));
          }
          bits = __bfloat16_as_ushort(__float2bfloat16_rn(old + bf16_round(y)));
        }
        const uint32_t other = __shfl_xor_sync(0xffffffffu, bits, 1);
        if (mine && !(wtid & 1))
          st_relaxed_u64(ph->ll_dst + ((row0 + wtid) >> 1), (static_cast<unsigned long long>(stamp) << 32) | (other << 16) | bits);
      }
    }
    if (tracing) trace_event(cx, wtid, EV_PHASE_DONE);
  }
  st.head = head;
  st.seq = seq;
  return ok;
}

// The same projection phase for every launch that is not the one-token row table.
//
// The weights are consumed by warp-level mma.sync (m16n8k16, bf16 in, fp32 out): one instruction
// multiplies 16 weight rows x 16 K-elements by up to eight token columns, where the CUDA-core loop
// this replaces needed 17 instructions per lane for 8 weights and kept the consumer warps, not HBM,
// the limit of a K loop.  A weight copy holds `kb` K chunks of the tile's rows, each chunk
// [rows][64] bf16 with the 128-byte swizzle (one three-dimensional TMA box); ldmatrix.x4 reads a
// 16 x 16 fragment from it without bank conflicts.  The eight warps split the K steps of a copy
// (warp w takes steps w, w + 8, ...) and keep fp32 accumulators for all row tiles of the unit; at
// the end of the unit the warps' partial sums meet in shared memory and are added in warp order.
// The token operand is bf16 in shared memory ([token][K], exact: every operand is a bf16 tensor in
// the reference), read as B fragments with two 32-bit loads per K step.
// Accumulation order depends only on the CTA's rotated chunk order: no dependence on timing.
template <int T, int NACC>
__device__ __noinline__ bool small_gemm_mma(const Ctx& cx, int gp, SmallState& st, int wtid, uint4 wu, int nch, uint32_t stamp) {
  const GemmPhase* ph = &cx.misc->phase[gp & 1];
  const int nunits = ph->nunits, rows = ph->rows, ksplit = ph->ksplit, kslice = ph->kslice, gran = ph->gran;
  const bool per_unit = ksplit > 1;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int kb = ph->kb;                          // K chunks per copy
  const int row_tiles = (rows + 15) >> 4;         // <= 4
  const uint32_t chunk_bytes = static_cast<uint32_t>(rows) * 128u;
  const int rot = k_rotation(cx.cta, cx.grid, kslice / kb) * kb;
  const uint32_t ring_base = smem_u32(cx.smem_a);
  const int ring_granules = cx.p->small_ring;
  // B fragment of this lane: token lane / 4, K elements 2 * (lane % 4) + {0, 1} and + 8 of a step
  const bool has_token = (lane >> 2) < T;
  const uint32_t x_lane = smem_u32(cx.smem_b) + (lane >> 2) * kXTokenBytes + (lane & 3) * 4;
  // A fragment: lane l addresses row (l % 8) + 8 * ((l / 8) % 2) of a row tile, 16-byte unit l / 16 of the step
  const uint32_t a_lane = static_cast<uint32_t>((lane & 7) + ((lane >> 3) & 1) * 8) * 128u;
  const uint32_t a_unit_kk = static_cast<uint32_t>((warp & 3) * 2 + (lane >> 4));
  const uint32_t x_lane_kk = x_lane + static_cast<uint32_t>(warp & 3) * 32u;
  float* part = reinterpret_cast<float*>(cx.smem_b + kPartOffset);
  int head = st.head, seq = st.seq;
  bool ok = true;
  if (cx.cta < nunits) {
    trace_event(cx, wtid, EV_PHASE_ENTER);
#pragma unroll 1
    for (int unit = cx.cta; unit < nunits; unit += cx.grid) {
      const int tile = unit / ksplit, slice = unit - tile * ksplit;
      if (per_unit || unit == cx.cta) {
        if (unit != cx.cta) small_sync();  // the previous unit has finished reading the operand
        // a normalising phase that opens a layer (or the lm_head) reads what the previous layer stamped
        if (ph->bmode == B_NORM) ok = small_stage_norm<false>(cx, ph, T, wtid, wu, (gp & 3) == 0 ? stamp - 1u : stamp) && ok;
        else ok = small_stage_cols<false>(cx, ph, slice * kslice, kslice, T, wtid, nch, stamp) && ok;
        small_sync();
        if (unit == cx.cta) trace_event(cx, wtid, EV_B_STAGED);
      }
      int seg, row0;
      tile_origin(ph, tile, seg, row0);
      // Two accumulator sets per row tile (K steps alternate between them), so that consecutive
      // mma.sync instructions do not wait for one another; they are added when the unit ends.
      float acc[NACC][4][2][4];
#pragma unroll
      for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[a][i][0][e] = acc[a][i][1][e] = 0.f;
      int slot = rot;
      // The K loop, instantiated per number of 16-row tiles: no branch inside, so the fragment loads of
      // a group of K steps issue back to back ahead of the MMAs.  A step past the copy's last one
      // re-reads the last step's fragment against a zero token operand.
      auto k_loop = [&](auto tiles_tag) {
        constexpr int RT = decltype(tiles_tag)::value;
        constexpr int U = RT == 1 ? 4 : 2;  // K steps in flight per warp
#pragma unroll 1
        for (int k0 = 0; k0 < kslice; k0 += kb) {
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            if (head + gran > ring_granules) head = 0;
            const uint32_t base = ring_base + head * kGranule;
            head += gran;
            const uint32_t bar = seq % kChunkBars;
            // After a failed wait the warp keeps walking the schedule without waiting, so that
            // every consumer still reaches the same block-wide barriers and leaves together.
            const bool got = ok && wait_mbar(cx, smem_u32(&cx.misc->full[bar]), (seq / kChunkBars) & 1, SITE_MMA_FULL, gp);
            ok = __all_sync(0xffffffffu, got);
            if (k0 == 0 && a == 0 && unit == cx.cta) trace_event(cx, wtid, EV_FIRST_COPY);
            // Warp w takes K steps w, w + 8, ...: the step inside a chunk (w % 4) is fixed, the chunk
            // advances by two per step, so a fragment address is the lane's constant plus chunk terms.
            const uint32_t x_copy = x_lane_kk + static_cast<uint32_t>(slot) * 128u;
            const uint32_t a_copy = base + a_lane;
#pragma unroll 1
            for (int c0 = warp >> 2; c0 < kb; c0 += 2 * U) {
              uint32_t bf[U][2], af[U][RT][4];
#pragma unroll
              for (int j = 0; j < U; ++j) {
                const int c = c0 + 2 * j;
                const bool live = has_token && c < kb;
                const uint32_t ce = static_cast<uint32_t>(min(c, kb - 1));
                bf[j][0] = live ? lds_u32(x_copy + ce * 128u) : 0u;
                bf[j][1] = live ? lds_u32(x_copy + ce * 128u + 16u) : 0u;
                const uint32_t chunk_addr = a_copy + ce * chunk_bytes;
                // the 128-byte swizzle exchanges the 16-byte units of a row by the row's position in its 1 KiB atom
                const uint32_t swz = (((chunk_addr >> 7) & 7u) ^ a_unit_kk) << 4;
#pragma unroll
                for (int i = 0; i < RT; ++i) ldmatrix_x4(af[j][i], chunk_addr + static_cast<uint32_t>(i) * 2048u + swz);
              }
#pragma unroll
              for (int j = 0; j < U; ++j)
#pragma unroll
                for (int i = 0; i < RT; ++i) mma_bf16_16816(acc[a][i][j & 1], af[j][i], bf[j][0], bf[j][1]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&cx.misc->empty[bar]));
            seq += 1;
          }
          slot = (slot + kb == kslice) ? 0 : slot + kb;
        }
      };
      switch (row_tiles) {
        case 1: k_loop(IntTag<1>{}); break;
        case 2: k_loop(IntTag<2>{}); break;
        case 3: k_loop(IntTag<3>{}); break;
        default: k_loop(IntTag<4>{}); break;
      }
#pragma unroll
      for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[a][i][0][e] += acc[a][i][1][e];
      if (unit == cx.cta) trace_event(cx, wtid, EV_FIRST_ACC);
      if (unit != cx.cta) small_sync();  // the previous unit's rows have been finished: `part` is free
      // D fragment: c0, c1 = row lane / 4, tokens 2 * (lane % 4) + {0, 1}; c2, c3 = eight rows further down
#pragma unroll
      for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = i * 16 + (lane >> 2) + (e >> 1) * 8;
            const int t = (lane & 3) * 2 + (e & 1);
            if (i < row_tiles && t < T) part[((warp * 2 + a) * kSmallTileRows + r) * kSplitTokens + t] = acc[a][i][0][e];
          }
      small_sync();
      {
        const bool mine = wtid < rows && row0 + wtid < ph->n[seg];
        uint32_t bits[T];
#pragma unroll
        for (int t = 0; t < T; ++t) bits[t] = 0u;
        if (mine) small_finish_row<T, false>(cx, ph, seg, slice, row0 + wtid, wtid, bits);
        if (ph->ll) {
          // Rows 2k and 2k + 1 (even tile height, even segment sizes) share a word:
          // {stamp, bf16 of the odd column, bf16 of the even column}, one 64-bit store.
          const int col = ph->out_col[seg] + row0 + wtid;
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const uint32_t other = __shfl_xor_sync(0xffffffffu, bits[t], 1);
            if (mine && !(wtid & 1))
              st_relaxed_u64(ph->ll_dst + static_cast<size_t>(t) * ph->ll_ld + (col >> 1),
                             (static_cast<unsigned long long>(stamp) << 32) | (other << 16) | bits[t]);
          }
        }
      }
    }
    trace_event(cx, wtid, EV_PHASE_DONE);
  }
  st.head = head;
  st.seq = seq;
  return ok;
}

template <int T, bool ROW>
__device__ __forceinline__ bool small_gemm_t(const Ctx& cx, int gp, SmallState& st, int wtid, uint4 wu, int nch,
                                             uint32_t stamp) {
  if constexpr (ROW) {  // one-token row table: CUDA-core consumer over plain rows
    if (cx.misc->phase[gp & 1].bulk) return small_gemm_rows(cx, gp, st, wtid, nch, stamp);
    return cx.misc->phase[gp & 1].nacc == 2 ? small_gemm<1, 2>(cx, gp, st, wtid, wu, nch, stamp)
                                            : small_gemm<1, 1>(cx, gp, st, wtid, wu, nch, stamp);
  } else {
    return cx.misc->phase[gp & 1].nacc == 2 ? small_gemm_mma<T, 2>(cx, gp, st, wtid, wu, nch, stamp)
                                            : small_gemm_mma<T, 1>(cx, gp, st, wtid, wu, nch, stamp);
  }
}

// Decode attention with RoPE, in-kernel KV append and a context split across
// CTAs; same arithmetic and rounding points as mk::attention_phase (scores
// bf16(q.k) * scale, fp32 softmax against the global max and sum of the row
// group, probabilities rounded to bf16, fp32 value sums; chunk partials are
// summed by the o-projection's operand staging).  Differences are in the order
// of the memory traffic only: the K rows of a unit are requested before q is
// rotated, the V rows before the softmax statistics are exchanged, so that one
// memory latency hides behind each of those steps.
struct SmallAttn {
  const unsigned long long* ll;    // stamped q/k/v words [batch][qkv width / 2], or null: read the bf16 buffer
  unsigned long long* out_ll;      // stamped fp32 chunk partials {stamp, fp32}, or null: att_part / out
  unsigned long long* out_pairs;   // with out_ll: the combined output as stamped bf16 pairs [batch][q_heads * hd / 2]
  const bf16* q; int q_ld;         // [batch][q_heads * hd] inside the qkv row
  bf16 *k, *v;                     // caches [batch][capacity][kv_heads][hd]
  long long kv_bstride; int kv_ld;
  const bf16 *knew, *vnew; int new_ld;
  bf16* out; int out_ld;           // [batch][q_heads * hd]
  int len;                         // filled positions before this call
  uint32_t stamp;
  float scale;
};

// Shared-memory plan of the attention phase inside the 64 KB activation region.
constexpr int kAttScoreBytes = 16 * 1024;   // fp32 scores [group][chunk]
constexpr int kAttTileBytes = 36 * 1024;    // one tile of cached K (then V) rows of the unit's head (288 keys of 64)
constexpr int kAttScratchBytes = 12 * 1024; // q (fp32 and bf16), cross-warp sums, new key/value, statistics
static_assert(kAttScoreBytes + kAttTileBytes + kAttScratchBytes <= kBBytes, "attention scratch exceeds its region");

// Code size matters here: every instruction of this function runs a handful of times per
// layer, so it is written as short loops (an unrolled version measured 128 KB of code and spent
// its time fetching instructions).  Rows of the cache go to shared memory with cp.async: no
// registers are tied up, and any number of keys can be in flight.
// Copy `count` rows of head_dim bf16 (row stride ld elements) into shared memory with cp.async,
// except row `skip` (the position being appended: its row is not in the cache yet).
__device__ __noinline__ void small_fetch_rows(uint32_t dst, const bf16* src, int ld, int count, int skip, int hd, int wtid) {
  const int shift = (hd == 64) ? 3 : 4;  // 16-byte pieces per row: 8 or 16
  const int total = count << shift;
#pragma unroll 1
  for (int it = wtid; it < total; it += kSmallWorkers) {
    const int key = it >> shift, piece = it & ((1 << shift) - 1);
    if (key != skip)  // piece p of row `key` lands at piece p ^ (key & 7): a column of pieces spreads over all banks
      cp_async16(dst + key * hd * 2 + ((piece ^ (key & 7)) << 4),
                 reinterpret_cast<const uint4*>(src + static_cast<long long>(key) * ld) + piece);
  }
}

template <bool use_mma>
__device__ __noinline__ bool small_attention(const Ctx& cx, const SmallAttn& A_in, int wtid, int nch) {
  // Private copies of everything this phase reads from the context, the parameters and its own arguments:
  // each poll and each barrier below is a compiler barrier for memory, behind which a value that lives
  // behind a reference would be loaded again (two dependent loads for a kernel parameter).
  const SmallAttn A = A_in;
  struct {
    int head_dim, q_heads, kv_heads, batch, qkv_ld, rope_style;
    const bf16 *cos_t, *sin_t;
    float *att_xch, *att_part;
  } p = {cx.p->head_dim, cx.p->q_heads, cx.p->kv_heads, cx.p->batch, cx.p->qkv_ld, cx.p->rope_style,
         cx.p->cos_t, cx.p->sin_t, cx.p->att_xch, cx.p->att_part};
  const int my_cta = cx.cta, grid = cx.grid;
  uint8_t* const region = cx.smem_b;
  const long long* const pos_s = cx.misc->pos_s;
  const int hd = p.head_dim, half = hd / 2;
  const int gs = p.q_heads / p.kv_heads;
  const int rows = p.batch * p.kv_heads;
  const int n_max = A.len + 1;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int lpk = hd / 8;    // lanes per key (16 B each)
  const int chunk = (n_max + nch - 1) / nch;
  const int units = rows * nch;
  const int tile_keys = kAttTileBytes / (hd * 2);
  const int row_bytes = hd * 2;

  float* sc = reinterpret_cast<float*>(region);                       // [gs][chunk]
  uint8_t* tile = region + kAttScoreBytes;                             // [tile_keys][hd] bf16
  float* qs = reinterpret_cast<float*>(tile + kAttTileBytes);             // [gs][hd]                4 KB
  float* red = qs + 8 * 128;                                              // [8 warps][128] / [parts][gs*hd]  4 KB
  bf16* kn = reinterpret_cast<bf16*>(red + kSmallWarps * 128);            // [hd]
  bf16* vn = kn + 128;                                                    // [hd]
  float* stat = reinterpret_cast<float*>(vn + 128);                       // [16]: max[8], sum[8]
  float* all = stat + 16;                                                 // [kMaxChunks][16]
  bf16* qb = reinterpret_cast<bf16*>(all + kMaxChunks * 16);              // [gs][hd]: q again as bf16 (exact)
  const uint32_t tile_addr = smem_u32(tile);
  // Both products run on the warp-level tensor cores: one mma.sync (m16n8k16) multiplies 16 cached
  // positions x 16 head dimensions by the (up to eight) query heads of the KV head, where a CUDA-core loop
  // needs 17 instructions per lane for eight elements; with eight warps per SM every instruction is ~8
  // cycles of this phase's latency chain.
  //   scores: D[16 keys][heads]  = K tile (ldmatrix)         x q[dims][heads]   (q fragments in registers)
  //   values: D[16 dims][heads] += V tile^T (ldmatrix.trans) x p[keys][heads]
  // Warps split the 16-key blocks (scores); for the values warp w takes dimension tile w % (hd / 16) and
  // every (8 * 16 / hd)-th key block, and the parts are added in part order.
  // (use_mma: a KV head with a single query head fills one of the eight MMA columns and measured 1.2 %
  // slower than the CUDA-core loops on the 1.7B shape; seven heads per group, Qwen2-0.5B, 8 % faster.  The
  // caller picks the instantiation by group size.)
  const int ksteps = hd / 16, dim_tiles = hd / 16;
  const int v_parts = kSmallWarps / dim_tiles > 0 ? kSmallWarps / dim_tiles : 1;   // 2 (hd 64) or 1 (hd 128)
  const int my_dt = warp % dim_tiles, my_part = warp / dim_tiles;
  const int lg = lane >> 2, lt = lane & 3;
  auto piece_addr = [&](int key, int piece) -> uint32_t {
    return tile_addr + key * row_bytes + ((piece ^ (key & 7)) << 4);
  };

#pragma unroll 1
  for (int u = my_cta; u < units; u += grid) {
    const int rowg = u / nch, ch = u - rowg * nch;
    const int b = rowg / p.kv_heads, kvh = rowg - b * p.kv_heads;
    const int j0 = ch * chunk;
    const int j1 = min(n_max, j0 + chunk);
    const int cl = max(0, j1 - j0);
    const int newpos = A.len;
    const bool owner = (A.len >= j0 && A.len < j1);
    const bf16* kbase = A.k + b * A.kv_bstride + kvh * hd;
    const bf16* vbase = A.v + b * A.kv_bstride + kvh * hd;
    const int ntiles = (cl + tile_keys - 1) / tile_keys;
    if (u != my_cta) small_sync();  // previous unit is done with the scratch

    // Copy keys [t0, t1) of `cache` (not the new position: its row is still in kn/vn) into the tile.
    auto fetch_tile = [&](const bf16* cache, int t0, int t1) {
      small_fetch_rows(tile_addr, cache + static_cast<long long>(t0) * A.kv_ld, A.kv_ld, t1 - t0, newpos - t0, hd, wtid);
    };
    fetch_tile(kbase, j0, min(j1, j0 + tile_keys));  // in flight while q is rotated

    // --- q of every head of the group and the new key (both rotated), and the new value: one round trip
    bool fresh = true;  // every stamped word this thread needs has arrived
    {
      const long long pos = pos_s[b];
      const int ropes = (gs + 1) * half;
      const int q_size = p.q_heads * hd, kv_size = p.kv_heads * hd;
      // Column c of sequence b's q/k/v row: from the bf16 buffer, or (small-launch table) from the word the
      // projection's epilogue stamped; waiting for the stamp is what orders this phase after that one.
      auto qkv_at = [&](int c) -> float {
        if (A.ll == nullptr) return ldcg_bf16(A.q + static_cast<long long>(b) * A.q_ld + c);
        const unsigned long long* word = A.ll + static_cast<size_t>(b) * (p.qkv_ld / 2) + (c >> 1);
        unsigned long long w = ld_relaxed_u64(word);
        uint32_t spins = 0;
        while (static_cast<uint32_t>(w >> 32) != A.stamp) {
          if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, -1 - rowg)) {
            fresh = false;
            break;
          }
          w = ld_relaxed_u64(word);
        }
        const uint32_t lo = static_cast<uint32_t>(w);
        return __uint_as_float((c & 1) ? (lo & 0xFFFF0000u) : (lo << 16));
      };
#pragma unroll 1
      for (int idx = wtid; idx < ropes + hd; idx += kSmallWorkers) {
        if (idx < ropes) {
          const int g = idx / half, i = idx - g * half;
          const int c0 = (g < gs) ? (kvh * gs + g) * hd : q_size + kvh * hd;
          float x1 = qkv_at(c0 + i);
          float x2 = qkv_at(c0 + i + half);
          const float cs = ldg_bf16(p.cos_t + pos * hd + i);
          const float sn = ldg_bf16(p.sin_t + pos * hd + i);
          rope_pair(x1, x2, cs, sn, p.rope_style, x1, x2);
          if (g < gs) {
            if constexpr (use_mma) {
              qb[g * hd + i] = __float2bfloat16_rn(x1);  // exact: both are bf16 values
              qb[g * hd + i + half] = __float2bfloat16_rn(x2);
            } else {
              qs[g * hd + i] = x1;
              qs[g * hd + i + half] = x2;
            }
          } else {
            kn[i] = __float2bfloat16_rn(x1);
            kn[i + half] = __float2bfloat16_rn(x2);
          }
        } else {
          const int i = idx - ropes;
          vn[i] = __float2bfloat16_rn(qkv_at(q_size + kv_size + kvh * hd + i));
        }
      }
    }
    cp_async_wait_all();
    if (!small_ok(cx, fresh)) return false;
    trace_event(cx, wtid, EV_ATT_INPUTS);
    uint32_t qfrag[8][2];  // B fragments: q[dims][query heads], one pair per 16 dimensions
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qfrag[ks][0] = qfrag[ks][1] = 0u;
      if (use_mma && ks < ksteps && lg < gs) {
        const bf16* at = qb + lg * hd + ks * 16 + lt * 2;
        qfrag[ks][0] = *reinterpret_cast<const uint32_t*>(at);
        qfrag[ks][1] = *reinterpret_cast<const uint32_t*>(at + 8);
      }
    }
    if (owner && newpos - j0 < tile_keys && wtid < lpk)  // the new key joins its tile (its row was not fetched)
      *reinterpret_cast<uint4*>(tile + (newpos - j0) * row_bytes + ((wtid ^ ((newpos - j0) & 7)) << 4)) =
          *reinterpret_cast<const uint4*>(kn + wtid * 8);
    if (owner) {  // in-kernel KV append
      bf16* kd = A.k + b * A.kv_bstride + static_cast<long long>(A.len) * A.kv_ld + kvh * hd;
      bf16* vd = A.v + b * A.kv_bstride + static_cast<long long>(A.len) * A.kv_ld + kvh * hd;
#pragma unroll 1
      for (int i = wtid; i < hd; i += kSmallWorkers) {
        kd[i] = kn[i];
        vd[i] = vn[i];
      }
    }

    // --- scores, tile by tile (one tile unless the chunk is longer than tile_keys)
#pragma unroll 1
    for (int t = 0; t < ntiles; ++t) {
      const int t0 = j0 + t * tile_keys, t1 = min(j1, t0 + tile_keys);
      if (t > 0) {
        small_sync();  // everyone is done with the previous tile
        fetch_tile(kbase, t0, t1);
        cp_async_wait_all();
        if (newpos >= t0 && newpos < t1 && wtid < lpk)
          *reinterpret_cast<uint4*>(tile + (newpos - t0) * row_bytes + ((wtid ^ ((newpos - t0) & 7)) << 4)) =
              *reinterpret_cast<const uint4*>(kn + wtid * 8);
        small_sync();
      } else {
        small_sync();  // the patched row of the first tile is visible
      }
      if constexpr (use_mma) {
      const int tk = t1 - t0;
#pragma unroll 1
        for (int blk = warp; blk * 16 < tk; blk += kSmallWarps) {
          float d[4] = {0.f, 0.f, 0.f, 0.f};
          const int row = blk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll 2
          for (int ks = 0; ks < ksteps; ++ks) {
            uint32_t af[4];
            ldmatrix_x4(af, piece_addr(row, ks * 2 + (lane >> 4)));
            mma_bf16_16816(d, af, qfrag[ks][0], qfrag[ks][1]);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = blk * 16 + lg + (e >> 1) * 8, n = lt * 2 + (e & 1);
            if (n < gs && key < tk) sc[n * chunk + (t0 - j0) + key] = bf16_round(d[e]) * A.scale;
          }
        }
      } else {
      // one thread per key: a 64- or 128-term fp32 chain per (key, head), no shuffles
#pragma unroll 1
        for (int key = wtid; key < t1 - t0; key += kSmallWorkers) {
          const int j = t0 + key;
          const uint8_t* krow = tile + key * row_bytes;
#pragma unroll 1
          for (int g = 0; g < gs; ++g) {
            const float* qv = qs + g * hd;
            // four partial sums (pieces 0, 4, ... / 1, 5, ... / ...): the same order as mk::attention_decode,
            // and a quarter of the dependent FMA chain
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
            sc[g * chunk + (j - j0)] = bf16_round(dot) * A.scale;
          }
        }
      }
    }
    small_sync();
    trace_event(cx, wtid, EV_ATT_SCORES);
    // --- the first tile of V rows replaces K: in flight while the statistics are built and exchanged
    fetch_tile(vbase, j0, min(j1, j0 + tile_keys));

    // --- chunk max, then chunk sum of exp(score - chunk max)
#pragma unroll 1
    for (int g = 0; g < gs; ++g) {
      float m = -INFINITY;
#pragma unroll 1
      for (int i = wtid; i < cl; i += kSmallWorkers) m = fmaxf(m, sc[g * chunk + i]);
      m = warp_max(m);
      if (lane == 0) red[warp * 8 + g] = m;
    }
    small_sync();
#pragma unroll 1
    for (int g = 0; g < gs; ++g) {
      float m = red[g];
#pragma unroll
      for (int w8 = 1; w8 < kSmallWarps; ++w8) m = fmaxf(m, red[w8 * 8 + g]);
      float sum = 0.f;
#pragma unroll 1
      for (int i = wtid; i < cl; i += kSmallWorkers) sum += expf(sc[g * chunk + i] - m);
      sum = warp_sum(sum);
      if (lane == 0) red[64 + warp * 8 + g] = sum;
      if (wtid == 0) stat[g] = m;
    }
    small_sync();
    if (wtid < gs) {
      float sum = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kSmallWarps; ++w8) sum += red[64 + w8 * 8 + wtid];
      stat[8 + wtid] = sum;
    }
    small_sync();

    if (nch > 1) {
      // --- publish (max, sum): every value travels with this phase's stamp in one 64-bit word,
      // so a reader that sees the stamp has the value (no fence, one round trip)
      unsigned long long* xch = reinterpret_cast<unsigned long long*>(p.att_xch) +
                                static_cast<size_t>(rowg) * kMaxChunks * (kExchangeFloats / 2);
      if (wtid < 16)
        st_relaxed_u64(xch + ch * (kExchangeFloats / 2) + wtid,
                       (static_cast<unsigned long long>(A.stamp) << 32) | __float_as_uint(stat[wtid]));
      bool ok = true;
      if (wtid < nch * 16) {
        const unsigned long long* theirs = xch + (wtid >> 4) * (kExchangeFloats / 2) + (wtid & 15);
        unsigned long long word = ld_relaxed_u64(theirs);
        uint32_t spins = 0;
        while (static_cast<uint32_t>(word >> 32) != A.stamp) {
          if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, rowg)) {
            ok = false;
            break;
          }
          word = ld_relaxed_u64(theirs);
        }
        all[wtid] = __uint_as_float(static_cast<uint32_t>(word));
      }
      if (!small_ok(cx, ok)) return false;
      if (wtid < gs) {
        float m = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < nch; ++c) m = fmaxf(m, all[c * 16 + wtid]);
        float sum = 0.f;
#pragma unroll 1
        for (int c = 0; c < nch; ++c) sum += all[c * 16 + 8 + wtid] * expf(all[c * 16 + wtid] - m);
        stat[wtid] = m;
        stat[8 + wtid] = sum;
      }
      small_sync();
    }

    trace_event(cx, wtid, EV_ATT_STATS);
    // --- probabilities (bf16, against the global max and sum)
#pragma unroll 1
    for (int g = 0; g < gs; ++g) {
      const float m = stat[g], denom = stat[8 + g];
#pragma unroll 1
      for (int i = wtid; i < cl; i += kSmallWorkers) sc[g * chunk + i] = bf16_round(expf(sc[g * chunk + i] - m) / denom);
    }
    const int cols = gs * hd;
    int parts;
    if constexpr (use_mma) {
    // --- value accumulation on the tensor cores; the parts' fp32 sums meet in `red` ([part][gs * hd])
      parts = v_parts;
      float vacc[4] = {0.f, 0.f, 0.f, 0.f};  // D[16 dims of tile my_dt][query heads]
#pragma unroll 1
      for (int t = 0; t < ntiles; ++t) {
        const int t0 = j0 + t * tile_keys, t1 = min(j1, t0 + tile_keys);
        if (t > 0) {
          small_sync();
          fetch_tile(vbase, t0, t1);
        }
        cp_async_wait_all();
        if (newpos >= t0 && newpos < t1 && wtid < lpk)  // the new value row joins its tile
          *reinterpret_cast<uint4*>(tile + (newpos - t0) * row_bytes + ((wtid ^ ((newpos - t0) & 7)) << 4)) =
              *reinterpret_cast<const uint4*>(vn + wtid * 8);
        const int tk = t1 - t0;
        if (tk & 15) {
          // the last 16-key block of a short tile: rows past the tile's keys meet zero probabilities, but what
          // the tile holds there must be finite for that product to be zero
          const int count = 16 - (tk & 15);
          for (int it = wtid; it < count * lpk; it += kSmallWorkers)
            *reinterpret_cast<uint4*>(tile + (tk + it / lpk) * row_bytes + ((it % lpk) << 4)) = make_uint4(0, 0, 0, 0);
        }
        small_sync();  // the tile has landed, and (first tile) the probabilities are complete
        if (my_part < parts) {
          const float* pr = sc + lg * chunk + (t0 - j0);
#pragma unroll 1
          for (int k16 = my_part; k16 * 16 < tk; k16 += parts) {
            // B fragment: probabilities of query head lane / 4 for keys 2 * (lane % 4) + {0, 1} and + 8 of the block
            const int key = k16 * 16 + lt * 2;
            float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
            if (lg < gs) {
              if (key < tk) p0 = pr[key];
              if (key + 1 < tk) p1 = pr[key + 1];
              if (key + 8 < tk) p2 = pr[key + 8];
              if (key + 9 < tk) p3 = pr[key + 9];
            }
            // A fragment: V^T from the tile's rows (keys): matrices (keys 0-7 | 8-15) x (dims 0-7 | 8-15) of the block
            const int row = k16 * 16 + (lane & 7) + (lane >> 4) * 8;
            uint32_t af[4];
            ldmatrix_x4_trans(af, piece_addr(row, my_dt * 2 + ((lane >> 3) & 1)));
            mma_bf16_16816(vacc, af, pack2(p0, p1), pack2(p2, p3));
          }
        }
      }
      if (my_part < parts) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = lt * 2 + (e & 1), d = my_dt * 16 + lg + (e >> 1) * 8;
          if (n < gs) red[my_part * cols + n * hd + d] = vacc[e];
        }
      }
    } else {
    // --- value accumulation: an item is (part of the keys, head of the group, 16-byte piece of the
      // output row); part p takes keys p, p + parts, ...; the fp32 sums of an item live in `red`
      // between tiles and for the final addition of the parts (parts * group * head_dim <= 1024 floats)
      const int pieces = gs * lpk;
      parts = kSmallWorkers / pieces;
      if (parts * cols > 1024) parts = 1024 / cols;
      if (parts < 1) parts = 1;
      const int items = parts * pieces;
#pragma unroll 1
      for (int t = 0; t < ntiles; ++t) {
        const int t0 = j0 + t * tile_keys, t1 = min(j1, t0 + tile_keys);
        if (t > 0) {
          small_sync();
          fetch_tile(vbase, t0, t1);
        }
        cp_async_wait_all();
        if (newpos >= t0 && newpos < t1 && wtid < lpk)  // the new value row joins its tile
          *reinterpret_cast<uint4*>(tile + (newpos - t0) * row_bytes + ((wtid ^ ((newpos - t0) & 7)) << 4)) =
              *reinterpret_cast<const uint4*>(vn + wtid * 8);
        small_sync();  // the tile has landed, and (first tile) the probabilities are complete
        const int tk = t1 - t0;
#pragma unroll 1
        for (int item = wtid; item < items; item += kSmallWorkers) {
          const int part = item / pieces, pc = item - part * pieces;
          const int g = pc / lpk, piece = pc - g * lpk;
          float* mine = red + (part * gs + g) * hd + piece * 8;
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = (t == 0) ? 0.f : mine[e];
          const float* pr = sc + g * chunk + (t0 - j0);
#pragma unroll 2
          for (int kk = part; kk < tk; kk += parts) {
            float vf[8];
            unpack8(*reinterpret_cast<const uint4*>(tile + kk * row_bytes + ((piece ^ (kk & 7)) << 4)), vf);
            const float w = pr[kk];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, vf[e], acc[e]);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) mine[e] = acc[e];
        }
      }
    }
    small_sync();
    trace_event(cx, wtid, EV_ATT_VALUES);
#pragma unroll 1
    for (int col = wtid; col < cols; col += kSmallWorkers) {
      float o = red[col];
#pragma unroll 1
      for (int part = 1; part < parts; ++part) o += red[part * cols + col];
      const int g = col / hd, d = col - g * hd;
      const int head = kvh * gs + g;
      if (A.out_ll != nullptr) {  // the o projection polls these words: no grid barrier in between
        const size_t row = static_cast<size_t>(b) * p.q_heads + head;
        st_relaxed_u64(A.out_ll + (row * kMaxChunks + ch) * hd + d,
                       (static_cast<unsigned long long>(A.stamp) << 32) | __float_as_uint(o));
      } else if (nch == 1) {
        A.out[static_cast<long long>(b) * A.out_ld + head * hd + d] = __float2bfloat16_rn(o);
      } else {
        const size_t row = static_cast<size_t>(b) * p.q_heads + head;
        __stcg(p.att_part + (row * kMaxChunks + ch) * hd + d, o);
      }
    }
    trace_event(cx, wtid, EV_ATT_PARTIAL);
    if (A.out_ll != nullptr && ch == 0) {
      // The first chunk's CTA adds the chunk partials of its heads in chunk order, rounds once and stamps the
      // result as bf16 pairs: the o projection then reads 4 bytes per output instead of 8 per chunk and output.
      bool fresh = true;
#pragma unroll 1
      for (int col0 = 0; col0 < cols; col0 += kSmallWorkers) {
        const int col = col0 + wtid;
        uint32_t bits = 0u;
        if (col < cols) {
          const int g = col / hd, d = col - g * hd;
          const size_t row = static_cast<size_t>(b) * p.q_heads + kvh * gs + g;
          float o = 0.f;
#pragma unroll 1
          for (int c = 0; c < nch; ++c)
            o += __uint_as_float(stamped_payload(cx, A.out_ll + (row * kMaxChunks + c) * hd + d, A.stamp, fresh));
          bits = __bfloat16_as_ushort(__float2bfloat16_rn(o));
        }
        const uint32_t other = __shfl_xor_sync(0xffffffffu, bits, 1);
        if (col < cols && !(col & 1))
          st_relaxed_u64(A.out_pairs + static_cast<size_t>(b) * (p.q_heads * hd / 2) + ((kvh * gs * hd + col) >> 1),
                         (static_cast<unsigned long long>(A.stamp) << 32) | (other << 16) | bits);
      }
      if (!small_ok(cx, fresh)) return false;
    }
  }
  return true;
}

// ---------------------------------------------------------------------------
// warp 0: weight producer of the small-launch kernel.  Same ring discipline as mk::producer_loop
// (FIFO reclaim of 1 KB granules, one full/empty barrier pair per copy in flight) without the
// streamed-operand and multi-token-tile cases, which this kernel never meets.
__device__ __noinline__ void small_producer(const Ctx& cx) {
  const KParams& p = *cx.p;
  const uint64_t policy = l2_policy_evict_first();
  // Everything below is read into registers once (per launch or per phase): each barrier wait is a compiler
  // barrier for memory, and a descriptor field read again behind it is a round trip to L2 in the one
  // thread whose pace decides how full the ring stays.
  const int ring_granules = p.small_ring, n_gemm = p.n_gemm;
  const GemmPhase* const table = p.phases;
  const int my_cta = cx.cta, grid = cx.grid;
  const uint32_t ring_base = smem_u32(cx.smem_a);
  const uint32_t full0 = smem_u32(&cx.misc->full[0]), empty0 = smem_u32(&cx.misc->empty[0]);
  uint8_t* const qstart = cx.misc->qstart;
  uint8_t* const qgran = cx.misc->qgran;
  int head = 0, seq = 0, oldest = 0;
  bool ok = true;
#pragma unroll 1
  for (int gp = 0; gp < n_gemm && ok; ++gp) {
    const GemmPhase* ph = table + gp;
    const int nacc = ph->nacc, gran = ph->gran, nunits = ph->nunits, ksplit = ph->ksplit, kslice = ph->kslice, kb = ph->kb;
    const int rows = ph->rows, nseg = ph->nseg, bulk = ph->bulk, rpc = ph->rpc, map3d = ph->map3d, k_elems = ph->k;
    const int ts1 = ph->tile_start[1], ts2 = ph->tile_start[2];
    const int n0 = ph->n[0], n1 = ph->n[1], n2 = ph->n[2];
    const CUtensorMap *m0 = ph->tmap[0], *m1 = ph->tmap[1], *m2 = ph->tmap[2];
    const bf16 *w0 = ph->w[0], *w1 = ph->w[1], *w2 = ph->w[2];
    const uint32_t bytes = static_cast<uint32_t>(rows) * 128u * static_cast<uint32_t>(kb);
    const int rot = k_rotation(my_cta, grid, kslice / kb) * kb;
#pragma unroll 1
    for (int unit = my_cta; unit < nunits && ok; unit += grid) {
      const int tile = unit / ksplit, slice = unit - tile * ksplit;
      // tile_origin() on the private copies
      int seg = 0;
      if (nacc == 1) {
        if (nseg > 1 && tile >= ts1) seg = 1;
        if (nseg > 2 && tile >= ts2) seg = 2;
      }
      const int row0 = (tile - (seg == 0 ? 0 : (seg == 1 ? ts1 : ts2))) * rows;
      const int kbase = slice * kslice;
      int k = rot;
      const int n_seg = seg == 0 ? n0 : (seg == 1 ? n1 : n2);
      const bf16* w_seg = seg == 0 ? w0 : (seg == 1 ? w1 : w2);
      const CUtensorMap* map_seg = seg == 0 ? m0 : (seg == 1 ? m1 : m2);
      const int tile_rows = min(rows, n_seg - row0);
      const int steps = bulk ? (tile_rows + rpc - 1) / rpc * kb : kslice * nacc;  // bulk: one step per copy
#pragma unroll 1
      for (int i = 0; i < steps && ok; i += kb) {
        const int a = (nacc == 2) ? ((i / kb) & 1) : 0;  // gate and up copies alternate
        const CUtensorMap* map = nacc == 2 ? (a ? m1 : m0) : map_seg;
        // Copies are consumed in issue order, so ring space is reclaimed by retiring the oldest copy in
        // flight until [lo, hi) is free; a copy never wraps, so the skipped tail is freed first.
        int lo = head, hi = head + gran;
        if (hi > ring_granules) hi = ring_granules;  // first the tail fragment, then (second trip) the slot at 0
#pragma unroll 1
        for (int trip = 0; trip < 2 && ok; ++trip) {
#pragma unroll 1
          while (oldest < seq) {
            const int os = qstart[oldest % kChunkBars], oe = os + qgran[oldest % kChunkBars];
            const bool overlaps = os < hi && lo < oe;
            if (!overlaps && seq - oldest < kChunkBars) break;
            if (!wait_mbar(cx, empty0 + (oldest % kChunkBars) * 8u, (oldest / kChunkBars) & 1, SITE_PRODUCER_EMPTY, gp)) {
              ok = false;
              break;
            }
            ++oldest;
          }
          if (head + gran <= ring_granules) break;  // no wrap: one trip
          head = 0;
          lo = 0;
          hi = gran;
        }
        if (!ok) break;
        const int start = head;
        head += gran;
        qstart[seq % kChunkBars] = static_cast<uint8_t>(start);
        qgran[seq % kChunkBars] = static_cast<uint8_t>(gran);
        const uint32_t full = full0 + (seq % kChunkBars) * 8u;
        const uint32_t dst = ring_base + start * kGranule;
        if (bulk) {  // rows [r, r + count) of the tile: whole rows, contiguous in memory
          const int r = i * rpc, count = min(rpc, tile_rows - r);
          const uint32_t copy_bytes = static_cast<uint32_t>(count) * static_cast<uint32_t>(k_elems) * 2u;
          mbar_expect_tx(full, copy_bytes);
          bulk_load_1d(dst, w_seg + static_cast<size_t>(row0 + r) * k_elems, copy_bytes, full, policy);
        } else if (map3d) {  // mma.sync consumer: 64 elements x the tile's rows x kb chunks, each chunk 128-byte swizzled
          mbar_expect_tx(full, bytes);
          tma_load_3d(dst, map, 0, row0, kbase + k, full, policy);
        } else {
          mbar_expect_tx(full, bytes);
          tma_load_2d(dst, map, (kbase + k) * kChunkK, row0, full, policy);
        }
        ++seq;
        if (nacc == 1 || a == 1) {
          k += kb;
          if (k == kslice) k = 0;
        }
      }
    }
  }
  if (!ok) {  // leaving early: every copy already issued must land before the CTA exits
    for (int i = max(0, seq - kChunkBars); i < seq; ++i) {
      const uint32_t bar = full0 + (i % kChunkBars) * 8u;
      for (uint32_t spins = 0; spins < (1u << 22); ++spins) {
        if (mbar_try_wait(bar, (i / kChunkBars) & 1)) break;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// consumers: whole-launch schedule (decode with the split-K phase table)


__device__ __forceinline__ uint4 small_norm_weight(const Ctx& cx, int gp, int wtid) {
  if (gp >= cx.misc->n_gemm) return make_uint4(0, 0, 0, 0);
  const GemmPhase* ph = &cx.misc->phase[gp & 1];
  if (ph->bmode != B_NORM || wtid >= ph->k / 8) return make_uint4(0, 0, 0, 0);
  return __ldg(reinterpret_cast<const uint4*>(ph->normw) + wtid);
}

// One projection phase; the next phase's descriptor is requested first and stored last.
template <int T, bool ROW>
__device__ __forceinline__ bool small_project(const Ctx& cx, SmallState& st, int gp, int nch, uint4 wu, int wtid,
                                              uint32_t stamp) {
  const uint32_t word = small_phase_word(cx, gp + 1, wtid);
  const bool ok = small_gemm_t<T, ROW>(cx, gp, st, wtid, wu, nch, stamp);
  small_phase_store(cx, gp + 1, wtid, word);
  return ok;
}

// Close a phase: arrive at the grid barrier, fetch what the next phase needs that no other CTA
// writes (its norm weight), wait.  `ok` is per warp on entry; the result is block-uniform.
__device__ __forceinline__ bool small_close(const Ctx& cx, SmallState& st, int next_gp, uint4& wu, bool ok, int wtid) {
  if (!ok) cx.misc->wabort = 1;
  small_arrive(cx, st, wtid);   // its bar.sync also publishes the prefetched descriptor to every consumer
  wu = small_norm_weight(cx, next_gp, wtid);
  return small_wait(cx, st, wtid);
}

// One kernel per token count: code that is compiled in but never runs still costs instruction-cache
// reach (a build with all four token counts in one kernel measured 8 % slower at one token).
template <int T, bool ROW>
__device__ void small_worker_loop(const Ctx& cx, int wtid) {
  const KParams& p = *cx.p;
  SmallState st;
  st.head = 0; st.seq = 0; st.passed = 0;
  const int q_size = p.q_heads * p.head_dim, kv_size = p.kv_heads * p.head_dim;
  const int gs = p.q_heads / p.kv_heads;
  SmallAttn A;
  A.ll = nullptr;
  A.out_ll = nullptr;
  A.out_pairs = nullptr;
  A.q = p.qkv; A.q_ld = p.qkv_ld;
  A.knew = p.qkv + q_size; A.vnew = A.knew + kv_size; A.new_ld = p.qkv_ld;
  A.out = p.attn; A.out_ld = q_size;
  A.kv_bstride = static_cast<long long>(p.capacity) * kv_size; A.kv_ld = kv_size;
  A.scale = p.att_scale;
  small_phase_store(cx, 0, wtid, small_phase_word(cx, 0, wtid));
  small_sync();
  uint4 wu = small_norm_weight(cx, 0, wtid);
  // One projection phase: the next descriptor is fetched while this phase runs.
  bool ok = true;  // per warp; made block-uniform by every close()
  auto project = [&](int gp, int nch) {
    ok = small_project<T, ROW>(cx, st, gp, nch, wu, wtid, p.att_epoch + static_cast<uint32_t>(gp >> 2) + 1u) && ok;
  };
  auto close = [&](int next_gp) -> bool { return small_close(cx, st, next_gp, wu, ok, wtid); };
  // The cached K and V rows of this CTA's attention units do not depend on this step: ask L2 for
  // them ahead of time (a (sequence, head) slice of the cache is 128-byte pieces 4 KB apart, slow
  // to fetch cold).  Layer 0 asks before its first phase; every later layer while the barrier that
  // closes the previous layer is pending, when the consumers have nothing else to do.
  auto prefetch_kv = [&](int layer) {
    if (layer >= p.layers) return;
    const int len = cx.misc->len_s[layer];
    const int nch = decode_chunks(len + 1, p.batch * p.kv_heads, cx.grid, gs, kAttScoreBytes);
    const int chunk = (len + 1 + nch - 1) / nch;
    const int units = p.batch * p.kv_heads * nch;
    const int shift = (p.head_dim == 64) ? 0 : 1;  // 128-byte lines per cached row of one head: 1 or 2
#pragma unroll 1
    for (int u = cx.cta; u < units; u += cx.grid) {
      const int rowg = u / nch, ch = u - rowg * nch;
      const int b = rowg / p.kv_heads, kvh = rowg - b * p.kv_heads;
      const int j0 = ch * chunk, j1 = min(len, j0 + chunk);
      const size_t head_off = static_cast<size_t>(b) * A.kv_bstride + static_cast<size_t>(kvh) * p.head_dim;
      const bf16* kb = static_cast<const bf16*>(p.kc[layer]) + head_off;
      const bf16* vb = static_cast<const bf16*>(p.vc[layer]) + head_off;
#pragma unroll 1
      for (int item = wtid; item < ((j1 - j0) << shift); item += kSmallWorkers) {
        const size_t off = static_cast<size_t>(j0 + (item >> shift)) * A.kv_ld + (item & shift) * 64;
        prefetch_l2(kb + off);
        prefetch_l2(vb + off);
      }
    }
  };
  prefetch_kv(0);
  if constexpr (ROW) {
    // One-token row table: every hand-off between phases travels as stamped words, so a layer needs no grid
    // barrier; block barriers only pass the shared memory from one phase to the next.
#pragma unroll 1
    for (int layer = 0; layer < p.layers; ++layer) {
      const int gp = layer * 4;
      project(gp, 1);                        // [RMSNorm of the stamped residual] q, k, v (+bias)
      if (!small_ok(cx, ok)) return;
      A.ll = p.qkv_ll;
      A.out_ll = p.att_ll;
      A.out_pairs = p.attn_ll;
      A.k = static_cast<bf16*>(p.kc[layer]); A.v = static_cast<bf16*>(p.vc[layer]);
      A.len = cx.misc->len_s[layer];
      A.stamp = p.att_epoch + static_cast<uint32_t>(layer) + 1u;
      const int nch = decode_chunks(A.len + 1, p.batch * p.kv_heads, cx.grid, gs, kAttScoreBytes);
      if (!(gs >= 2 ? small_attention<true>(cx, A, wtid, nch) : small_attention<false>(cx, A, wtid, nch))) return;
      trace_event(cx, wtid, EV_ATTENTION_DONE);
      if (!small_ok(cx, ok)) return;
      project(gp + 1, nch);                  // o_proj rows + residual -> stamped residual
      if (!small_ok(cx, ok)) return;
      wu = small_norm_weight(cx, gp + 2, wtid);
      project(gp + 2, 1);                    // [RMSNorm] gate, up -> SiLU*up, stamped
      if (!small_ok(cx, ok)) return;
      project(gp + 3, 1);                    // down rows + residual -> stamped residual
      prefetch_kv(layer + 1);
      if (!small_ok(cx, ok)) return;
      wu = small_norm_weight(cx, gp + 4, wtid);
    }
    project(p.layers * 4, 1);                // [final RMSNorm] lm_head
    // the only grid barrier: every CTA has read the valid lengths (in its prologue) before they move on
    if (!ok) cx.misc->wabort = 1;
    small_arrive(cx, st, wtid);
    if (!small_wait(cx, st, wtid)) return;
    if (cx.cta == 0)
      for (int layer = wtid; layer < p.layers; layer += kSmallWorkers) *p.len[layer] = cx.misc->len_s[layer] + 1;
    if (p.sample) greedy_sample<1, kSmallWorkers>(cx, wtid, reinterpret_cast<float*>(cx.smem_b));
    return;
  } else {
  for (int layer = 0; layer < p.layers; ++layer) {
    const int gp = layer * 4;
    const bool handoff = cx.misc->phase[gp & 1].ll != 0;  // same for every layer and CTA
    project(gp, 1);                          // [residual update, RMSNorm] q, k, v (+bias)
    if (handoff) {
      // q/k/v travel as stamped words: attention starts as soon as this CTA's own tile is out and waits
      // word by word for the rows of its head; only the shared memory has to be handed over.
      A.ll = p.qkv_ll;
      A.out_ll = p.att_ll;
      A.out_pairs = p.attn_ll;
      if (!small_ok(cx, ok)) return;
    } else if (!close(gp + 1)) {
      return;
    }
    A.k = static_cast<bf16*>(p.kc[layer]); A.v = static_cast<bf16*>(p.vc[layer]);
    A.len = cx.misc->len_s[layer];
    A.stamp = p.att_epoch + static_cast<uint32_t>(layer) + 1u;
    const int nch = decode_chunks(A.len + 1, p.batch * p.kv_heads, cx.grid, gs, kAttScoreBytes);
    if (!(gs >= 2 ? small_attention<true>(cx, A, wtid, nch) : small_attention<false>(cx, A, wtid, nch))) return;       // RoPE, KV append, split-context attention
    trace_event(cx, wtid, EV_ATTENTION_DONE);
    if (handoff) {
      if (!small_ok(cx, ok)) return;         // the o projection polls the stamped attention partials
    } else {
      if (!close(gp + 1)) return;
      if (cx.cta == 0 && wtid == 0) *p.len[layer] = A.len + 1;  // publish after the interval closes
    }
    project(gp + 1, nch);                    // o_proj (fp32 K-slice partials)
    if (!close(gp + 2)) return;
    if (handoff && cx.cta == 0 && wtid == 0) *p.len[layer] = A.len + 1;  // every attention unit is long done
    project(gp + 2, 1);                      // [residual update, RMSNorm] gate, up -> SiLU*up
    if (handoff) {
      if (!small_ok(cx, ok)) return;         // the down projection polls the stamped activations
    } else if (!close(gp + 3)) {
      return;
    }
    project(gp + 3, 1);                      // down (fp32 K-slice partials)
    {  // the barrier that closes the layer, with the next layer's cache prefetch between its halves
      if (!ok) cx.misc->wabort = 1;
      small_arrive(cx, st, wtid);
      wu = small_norm_weight(cx, gp + 4, wtid);
      prefetch_kv(layer + 1);
      if (!small_wait(cx, st, wtid)) return;
    }
  }
  project(p.layers * 4, 1);                               // [residual update, final RMSNorm] lm_head
  if (p.sample) {  // one more grid barrier: every CTA's logits are out and nobody reads the ids any more
    if (!ok) cx.misc->wabort = 1;
    small_arrive(cx, st, wtid);
    if (!small_wait(cx, st, wtid)) return;
    greedy_sample<1, kSmallWorkers>(cx, wtid, reinterpret_cast<float*>(cx.smem_b));
  }
  }
}

// ---------------------------------------------------------------------------
// the kernel

template <int T, bool ROW>
__global__ void __launch_bounds__(kSmallThreads, 1) megakernel_small(const __grid_constant__ KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctx cx;
  cx.p = &p;
  cx.ctrl = p.ctrl;
  cx.smem_a = smem;
  cx.smem_b = smem + p.small_ring * kGranule;
  cx.misc = reinterpret_cast<SmemMisc*>(cx.smem_b + kBBytes);
  cx.tc = nullptr;
  cx.deadline = clock64() + p.timeout_cycles;
  cx.cta = blockIdx.x;
  cx.grid = gridDim.x;
  const int tid = threadIdx.x, warp = tid >> 5;

  if (tid == 0) {
    for (int s = 0; s < kChunkBars; ++s) {
      mbar_init(smem_u32(&cx.misc->full[s]), 1);
      mbar_init(smem_u32(&cx.misc->empty[s]), kSmallWarps);  // one arrival per consumer warp
    }
    cx.misc->wabort = 0;
    cx.misc->bad = 0;
    cx.misc->flag = 0;
    cx.misc->trace_n = 0;
    cx.misc->trace_on = p.trace_cap != 0;
    cx.misc->n_gemm = p.n_gemm;
    cx.misc->epoch = p.epoch;
    cx.misc->phases = p.phases;
    mbar_fence_init();
  }
  __syncthreads();
  // Prologue validation (same inputs in every CTA, so the verdict is grid-uniform); the
  // positions and the valid lengths as they are before this call stay in shared memory.
  {
    int bad = 0;
    for (int t = tid; t < p.m; t += kSmallThreads) {
      const long long id = p.ids[t];
      long long pos = p.pos[t];
      if (id < 0 || id >= p.embed_rows || pos < 0 || pos >= p.max_positions) {
        bad = MK_STATUS_BAD_INDEX;
        pos = 0;
      }
      cx.misc->pos_s[t] = pos;
    }
    for (int l = tid; l < p.layers; l += kSmallThreads) {
      const int len = *p.len[l];
      if (len < 0 || len + 1 > p.capacity) bad = MK_STATUS_KV_OVERFLOW;
      cx.misc->len_s[l] = len;
    }
    if (bad) atomicMax(&cx.misc->bad, bad);
  }
  __syncthreads();
  const int bad = *reinterpret_cast<volatile int*>(&cx.misc->bad);
  if (bad) {
    refuse_outputs(cx, bad, tid, kSmallThreads);
  } else if (warp == 0) {
    if (tid == 0) small_producer(cx);
  } else {
    small_worker_loop<T, ROW>(cx, tid - 32);
  }
}

}  // namespace mk
