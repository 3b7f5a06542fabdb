// The decode megakernel for launches of at most four tokens (batch-1 decode is
// the case that matters): same phase tables, weight ring, TMA producer and
// consumer-side split-K reduction as mk::megakernel, but the weight tiles are
// consumed by CUDA-core FMAs.
//
// Why not the tensor core here: one tcgen05.mma of 128 weight rows by 16 token
// columns occupies the tensor pipe for ~78 cycles whatever the token count and
// however few of the 128 rows hold weights (an even split of a projection over
// 148 CTAs wants tiles of 42-56 rows), which capped a CTA at 6-12 bytes of
// weights per cycle where HBM can deliver 22.  A matrix-vector product needs
// one FMA per weight and token: eight consumer warps read the TMA-filled ring
// slots with 16-byte shared loads (eight lanes share a weight row, 32 rows per
// pass), which is about 80 issue slots per 7 KB chunk and token.
//
// Roles: warp 0 = TMA producer (mk::producer_loop, unchanged), warps 1-8 =
// consumers (operand staging with the RMSNorm and the pending residual update
// fused in, FMA projection, epilogue, decode attention, grid barriers).  No
// TMEM, no MMA warp.  Everything that can be fetched before a grid barrier
// opens (phase descriptor, norm weights, K rows of the cache) is fetched there.
#pragma once
#include "decoder_kernel.cuh"

namespace mk {

constexpr int kSmallWarps = 8;
constexpr int kSmallWorkers = kSmallWarps * 32;
constexpr int kSmallThreads = 32 + kSmallWorkers;
constexpr int kXFloats = kBSlots * kChunkK;  // activation operand of one K slice per token, fp32
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
    const uint32_t target = cx.p->epoch + st.passed * static_cast<uint32_t>(cx.grid);
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

__device__ __forceinline__ void small_prefetch_phase(const Ctx& cx, int gp, int wtid) {
  if (gp >= cx.p->n_gemm) return;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(cx.p->phases + gp);
  uint32_t* dst = reinterpret_cast<uint32_t*>(&cx.misc->phase[gp & 1]);
  if (wtid < static_cast<int>(sizeof(GemmPhase) / 4)) dst[wtid] = __ldg(src + wtid);
}
static_assert(sizeof(GemmPhase) / 4 <= kSmallWorkers, "one word of the phase descriptor per consumer thread");

// fp32 operand layout: per token kXFloats floats; inside a 64-element K chunk the
// eight 8-element vectors are stored as two float4 halves, 128 bytes apart, so
// that the eight lanes sharing a weight row read 128 contiguous bytes per load.
__device__ __forceinline__ float* x_slot(const Ctx& cx, int t, int chunk, int vec) {
  return reinterpret_cast<float*>(cx.smem_b) + t * kXFloats + chunk * kChunkK + vec * 4;
}
__device__ __forceinline__ void x_store(const Ctx& cx, int t, int chunk, int vec, const float* f) {
  float* dst = x_slot(cx, t, chunk, vec);
  *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(dst + 32) = make_float4(f[4], f[5], f[6], f[7]);
}

// RMSNorm fused with staging (K = hidden <= 2048: one 8-element vector per
// thread and token).  Also applies the pending residual update of the split-K
// table: x = residual + bf16(sum of the previous projection's fp32 K-slice
// partials, in slice order), writes this CTA's share of x back as the new
// residual stream, and normalises x with the two roundings of the Hugging Face
// RMSNorm.  `wu` is this thread's vector of the norm weight, loaded by the
// caller before the grid barrier opened.
__device__ __noinline__ void small_stage_norm(const Ctx& cx, const GemmPhase* ph, int mt, int wtid, uint4 wu) {
  const KParams& p = *cx.p;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int nvec = ph->k / 8;
  const int parts = ph->add_parts;
  const int writers = min(cx.grid, ph->nunits);
  const bool active = wtid < nvec;
  float w[8];
  unpack8(wu, w);
  for (int t = 0; t < mt; ++t) {
    float f[8];
    uint4 xu = make_uint4(0, 0, 0, 0);
    if (active) {
      const uint4* row = reinterpret_cast<const uint4*>(activation_row(p, ph, t));
      xu = __ldcg(row + wtid);
      float4 lo[kMaxSplit], hi[kMaxSplit];
#pragma unroll
      for (int s8 = 0; s8 < kMaxSplit; ++s8) {
        if (s8 < parts) {
          const float4* part = reinterpret_cast<const float4*>(ph->partial + (static_cast<size_t>(s8) * p.m + t) * ph->k) + wtid * 2;
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
      if (ph->h_out && (wtid * writers) / nvec == cx.cta)
        __stcg(reinterpret_cast<uint4*>(ph->h_out + static_cast<size_t>(t) * ph->k) + wtid, xu);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) sum = fmaf(f[e], f[e], sum);
    sum = warp_sum(sum);
    if (lane == 0) cx.misc->sred[t][warp] = sum;
    small_sync();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kSmallWarps; ++i) total += cx.misc->sred[t][i];
    const float r = 1.0f / sqrtf(total / static_cast<float>(ph->k) + p.eps);
    if (active) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = bf16_round(w[e] * bf16_round(f[e] * r));
      x_store(cx, t, wtid >> 3, wtid & 7, f);
    }
  }
}

// Plain or attention-output operand: K chunks [k0, k0 + count) of every token.
__device__ __noinline__ void small_stage_cols(const Ctx& cx, const GemmPhase* ph, int k0, int count, int mt, int wtid,
                                              int nch) {
  const KParams& p = *cx.p;
  const int per_token = count * 8;
  const int items = per_token * mt;
  for (int item0 = wtid; item0 < items; item0 += kSmallWorkers * 4) {
    uint4 u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int item = item0 + i * kSmallWorkers;
      if (item < items) {
        const int t = item / per_token, rem = item - t * per_token;
        const int col = (k0 + (rem >> 3)) * kChunkK + (rem & 7) * 8;
        u[i] = (ph->bmode == B_ATTN) ? attention_vec(p, t, col, nch)
                                     : __ldcg(reinterpret_cast<const uint4*>(activation_row(p, ph, t) + col));
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int item = item0 + i * kSmallWorkers;
      if (item < items) {
        const int t = item / per_token, rem = item - t * per_token;
        float f[8];
        unpack8(u[i], f);
        x_store(cx, t, rem >> 3, rem & 7, f);
      }
    }
  }
}

// Projection phase gp for this CTA's units.  The caller has made the phase
// descriptor visible in cx.misc->phase[gp & 1]; `wu` is the norm-weight vector
// for B_NORM phases.  Accumulation order per output: lane c of the row's eight
// lanes sums elements [8c, 8c+8) of every K chunk in the CTA's rotated chunk
// order, then a fixed shuffle tree adds the eight lanes: no dependence on timing.
template <int T, int NACC>
__device__ __noinline__ bool small_gemm(const Ctx& cx, int gp, SmallState& st, int wtid, uint4 wu, int nch) {
  const GemmPhase* ph = &cx.misc->phase[gp & 1];
  const int nunits = ph->nunits, rows = ph->rows, ksplit = ph->ksplit, kslice = ph->kslice, gran = ph->gran;
  const bool per_unit = ksplit > 1;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int c = lane & 7, rsub = lane >> 3;
  const int kb = ph->kb;                 // K chunks per weight copy; a slot holds [rows][kb * 64] bf16, unswizzled
  const int lane_row = warp * 4 + rsub;  // row inside a 32-row pass
  const uint32_t row_bytes = static_cast<uint32_t>(kb) * 128u;
  const uint32_t lane_off = lane_row * row_bytes + (c << 4);
  const uint32_t pass_bytes = 32u * row_bytes;
  const int passes = (rows + 31) >> 5;
  const int rot = k_rotation(cx.cta, cx.grid, kslice / kb) * kb;
  const uint32_t ring_base = smem_u32(cx.smem_a);
  const uint32_t x_base = smem_u32(cx.smem_b) + c * 16;
  int head = st.head, seq = st.seq;
  bool ok = true;
  if (cx.cta < nunits) {
    trace_event(cx, wtid, EV_PHASE_ENTER);
    for (int unit = cx.cta; unit < nunits; unit += cx.grid) {
      const int tile = unit / ksplit, slice = unit - tile * ksplit;
      if (per_unit || unit == cx.cta) {
        if (unit != cx.cta) small_sync();  // the previous unit has finished reading the operand
        if (ph->bmode == B_NORM) small_stage_norm(cx, ph, T, wtid, wu);
        else small_stage_cols(cx, ph, slice * kslice, kslice, T, wtid, nch);
        small_sync();
        if (unit == cx.cta) trace_event(cx, wtid, EV_B_STAGED);
      }
      int seg, row0;
      tile_origin(ph, tile, seg, row0);
      // bias of this lane's rows, fetched before the K loop
      float bias_v[4] = {0.f, 0.f, 0.f, 0.f};
      if (ph->epi == EPI_STORE && ph->bias[seg] && c == 0) {
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {
          const int r = ps * 32 + lane_row;
          if (ps < passes && r < rows && row0 + r < ph->n[seg]) bias_v[ps] = ldg_bf16(ph->bias[seg] + row0 + r);
        }
      }
      float acc[NACC][4][T];
#pragma unroll
      for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int ps = 0; ps < 4; ++ps)
#pragma unroll
          for (int t = 0; t < T; ++t) acc[a][ps][t] = 0.f;
      int slot = rot;
      for (int i = 0; i < kslice; i += kb) {
        uint32_t base[NACC];
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
          if (head + gran > kRingGranules) head = 0;
          base[a] = ring_base + head * kGranule + lane_off;
          head += gran;
          const uint32_t bar = (seq + a) % kChunkBars;
          // After a failed wait the warp keeps walking the schedule without waiting, so that
          // every consumer still reaches the same block-wide barriers and leaves together.
          const bool got = ok && wait_mbar(cx, smem_u32(&cx.misc->full[bar]), ((seq + a) / kChunkBars) & 1, SITE_MMA_FULL, gp);
          ok = __all_sync(0xffffffffu, got);
        }
        for (int j = 0; j < kb; ++j) {
          float xf[T][8];
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const uint4 lo = lds_v4(x_base + (t * kXFloats + (slot + j) * kChunkK) * 4);
            const uint4 hi = lds_v4(x_base + (t * kXFloats + (slot + j) * kChunkK + 32) * 4);
            xf[t][0] = __uint_as_float(lo.x); xf[t][1] = __uint_as_float(lo.y);
            xf[t][2] = __uint_as_float(lo.z); xf[t][3] = __uint_as_float(lo.w);
            xf[t][4] = __uint_as_float(hi.x); xf[t][5] = __uint_as_float(hi.y);
            xf[t][6] = __uint_as_float(hi.z); xf[t][7] = __uint_as_float(hi.w);
          }
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
#pragma unroll
            for (int ps = 0; ps < 4; ++ps) {
              if (ps < passes) {
                float wf[8];
                unpack8(lds_v4(base[a] + ps * pass_bytes + j * 128), wf);
#pragma unroll
                for (int t = 0; t < T; ++t)
#pragma unroll
                  for (int e = 0; e < 8; ++e) acc[a][ps][t] = fmaf(wf[e], xf[t][e], acc[a][ps][t]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int a = 0; a < NACC; ++a) mbar_arrive(smem_u32(&cx.misc->empty[(seq + a) % kChunkBars]));
        }
        seq += NACC;
        slot = (slot + kb == kslice) ? 0 : slot + kb;
      }
      if (unit == cx.cta) trace_event(cx, wtid, EV_FIRST_ACC);
#pragma unroll
      for (int ps = 0; ps < 4; ++ps) {
        if (ps < passes) {
          float v[2][T];
#pragma unroll
          for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int t = 0; t < T; ++t) {
              float x = acc[a][ps][t];
              x += __shfl_xor_sync(0xffffffffu, x, 1);
              x += __shfl_xor_sync(0xffffffffu, x, 2);
              x += __shfl_xor_sync(0xffffffffu, x, 4);
              v[a][t] = x;
            }
          const int r = ps * 32 + lane_row;
          const int n = row0 + r;
          if (c == 0 && r < rows && n < ph->n[seg]) {
            if (ph->epi == EPI_PARTIAL) {
              store_partial<T>(cx, ph, slice, n, v[0], 0, T);
            } else {
              float pre[T];
              pre[0] = bias_v[ps];
              if (ph->epi == EPI_RESIDUAL) epilogue_prefetch<T>(cx, ph, seg, n, 0, T, pre);
              apply_epilogue<T>(cx, ph, seg, n, v, pre, 0, T);
            }
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

template <int T>
__device__ __forceinline__ bool small_gemm_t(const Ctx& cx, int gp, SmallState& st, int wtid, uint4 wu, int nch) {
  return cx.misc->phase[gp & 1].nacc == 2 ? small_gemm<T, 2>(cx, gp, st, wtid, wu, nch)
                                          : small_gemm<T, 1>(cx, gp, st, wtid, wu, nch);
}

__device__ __forceinline__ bool small_gemm_any(const Ctx& cx, int gp, SmallState& st, int wtid, uint4 wu, int nch) {
  switch (cx.p->m) {
    case 1: return small_gemm_t<1>(cx, gp, st, wtid, wu, nch);
    case 2: return small_gemm_t<2>(cx, gp, st, wtid, wu, nch);
    case 3: return small_gemm_t<3>(cx, gp, st, wtid, wu, nch);
    default: return small_gemm_t<4>(cx, gp, st, wtid, wu, nch);
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
  const bf16* q; int q_ld;         // [batch][q_heads * hd] inside the qkv row
  bf16 *k, *v;                     // caches [batch][capacity][kv_heads][hd]
  long long kv_bstride; int kv_ld;
  const bf16 *knew, *vnew; int new_ld;
  bf16* out; int out_ld;           // [batch][q_heads * hd]
  int len;                         // filled positions before this call
  uint32_t stamp;
  float scale;
};

__device__ __noinline__ bool small_attention(const Ctx& cx, const SmallAttn& A, int wtid, int nch) {
  const KParams& p = *cx.p;
  const int hd = p.head_dim, half = hd / 2;
  const int gs = p.q_heads / p.kv_heads;
  const int rows = p.batch * p.kv_heads;
  const int n_max = A.len + 1;
  const int warp = wtid >> 5, lane = wtid & 31;
  const int lpk = hd / 8;    // lanes per key (16 B each)
  const int kpw = 32 / lpk;  // keys per warp pass
  const int sub = lane / lpk, dg = lane % lpk;
  const int chunk = (n_max + nch - 1) / nch;
  const int units = rows * nch;
  constexpr int kU = 8;
  const int pass = kSmallWarps * kpw;

  float* sc = reinterpret_cast<float*>(cx.smem_b);                // [gs][chunk]
  float* qs = reinterpret_cast<float*>(cx.smem_b + kScoreBytes);  // [gs][hd]
  float* red = qs + 8 * 128;                                      // [8][128]
  bf16* kn = reinterpret_cast<bf16*>(red + kSmallWarps * 128);    // [hd]
  bf16* vn = kn + 128;                                            // [hd]
  float* stat = reinterpret_cast<float*>(vn + 128);               // [16]: max[8], sum[8]

  for (int u = cx.cta; u < units; u += cx.grid) {
    const int rowg = u / nch, ch = u - rowg * nch;
    const int b = rowg / p.kv_heads, kvh = rowg - b * p.kv_heads;
    const int j0 = ch * chunk;
    const int j1 = min(n_max, j0 + chunk);
    const int cl = max(0, j1 - j0);
    const int newpos = A.len;
    const bool owner = (A.len >= j0 && A.len < j1);
    const bf16* kbase = A.k + b * A.kv_bstride + kvh * hd;
    const bf16* vbase = A.v + b * A.kv_bstride + kvh * hd;
    if (u != cx.cta) small_sync();  // previous unit is done with the scratch

    // --- first batch of cached K rows: in flight while q is rotated
    uint4 ku[kU];
#pragma unroll
    for (int u8 = 0; u8 < kU; ++u8) {
      const int j = j0 + warp * kpw + u8 * pass + sub;
      ku[u8] = make_uint4(0, 0, 0, 0);
      if (j < j1 && j != newpos) ku[u8] = __ldcg(reinterpret_cast<const uint4*>(kbase + static_cast<long long>(j) * A.kv_ld) + dg);
    }
    // --- q of every head of the group, the new key (both rotated) and the new value
    const long long pos = cx.misc->pos_s[b];
    for (int idx = wtid; idx < (gs + 1) * half; idx += kSmallWorkers) {
      const int g = idx / half, i = idx - g * half;
      const bf16* src = (g < gs) ? A.q + static_cast<long long>(b) * A.q_ld + (kvh * gs + g) * hd
                                 : A.knew + static_cast<long long>(b) * A.new_ld + kvh * hd;
      float first = ldcg_bf16(src + i);
      float second = ldcg_bf16(src + i + half);
      const float cs = ldg_bf16(p.cos_t + pos * hd + i);
      const float sn = ldg_bf16(p.sin_t + pos * hd + i);
      rope_pair(first, second, cs, sn, p.rope_style, first, second);
      if (g < gs) {
        qs[g * hd + i] = first;
        qs[g * hd + i + half] = second;
      } else {
        kn[i] = __float2bfloat16_rn(first);
        kn[i + half] = __float2bfloat16_rn(second);
      }
    }
    for (int i = wtid; i < hd; i += kSmallWorkers)
      vn[i] = __float2bfloat16_rn(ldcg_bf16(A.vnew + static_cast<long long>(b) * A.new_ld + kvh * hd + i));
    small_sync();
    if (owner) {  // in-kernel KV append
      bf16* kd = A.k + b * A.kv_bstride + static_cast<long long>(A.len) * A.kv_ld + kvh * hd;
      bf16* vd = A.v + b * A.kv_bstride + static_cast<long long>(A.len) * A.kv_ld + kvh * hd;
      for (int i = wtid; i < hd; i += kSmallWorkers) {
        kd[i] = kn[i];
        vd[i] = vn[i];
      }
    }

    // --- scores
    for (int base = j0 + warp * kpw; base < j1; base += pass * kU) {
      if (base != j0 + warp * kpw) {
#pragma unroll
        for (int u8 = 0; u8 < kU; ++u8) {
          const int j = base + u8 * pass + sub;
          ku[u8] = make_uint4(0, 0, 0, 0);
          if (j < j1 && j != newpos) ku[u8] = __ldcg(reinterpret_cast<const uint4*>(kbase + static_cast<long long>(j) * A.kv_ld) + dg);
        }
      }
#pragma unroll
      for (int u8 = 0; u8 < kU; ++u8) {
        if (base + u8 * pass >= j1) break;  // warp-uniform
        const int j = base + u8 * pass + sub;
        if (j == newpos) ku[u8] = *reinterpret_cast<const uint4*>(kn + dg * 8);
        float kf[8];
        unpack8(ku[u8], kf);
        for (int g = 0; g < gs; ++g) {
          const float* qv = qs + g * hd + dg * 8;
          float dot = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(qv[e], kf[e], dot);
          for (int o = 1; o < lpk; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          if (dg == 0 && j < j1) sc[g * chunk + (j - j0)] = bf16_round(dot) * A.scale;
        }
      }
    }
    // --- first batch of V rows: in flight while the statistics are built and exchanged
    uint4 vu[kU];
#pragma unroll
    for (int u8 = 0; u8 < kU; ++u8) {
      const int j = j0 + warp * kpw + u8 * pass + sub;
      vu[u8] = make_uint4(0, 0, 0, 0);
      if (j < j1 && j != newpos) vu[u8] = __ldcg(reinterpret_cast<const uint4*>(vbase + static_cast<long long>(j) * A.kv_ld) + dg);
    }
    small_sync();

    // --- chunk max, then chunk sum of exp(score - chunk max)
    for (int g = 0; g < gs; ++g) {
      float m = -INFINITY;
      for (int i = wtid; i < cl; i += kSmallWorkers) m = fmaxf(m, sc[g * chunk + i]);
      m = warp_max(m);
      if (lane == 0) red[warp * 8 + g] = m;
    }
    small_sync();
    for (int g = 0; g < gs; ++g) {
      float m = red[g];
#pragma unroll
      for (int w8 = 1; w8 < kSmallWarps; ++w8) m = fmaxf(m, red[w8 * 8 + g]);
      float s = 0.f;
      for (int i = wtid; i < cl; i += kSmallWorkers) s += expf(sc[g * chunk + i] - m);
      s = warp_sum(s);
      if (lane == 0) red[64 + warp * 8 + g] = s;
      if (wtid == 0) stat[g] = m;
    }
    small_sync();
    if (wtid < gs) {
      float s = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kSmallWarps; ++w8) s += red[64 + w8 * 8 + wtid];
      stat[8 + wtid] = s;
    }
    small_sync();

    if (nch > 1) {
      // --- publish (max, sum) with this phase's stamp; wait for every chunk of the row group
      float* mine = p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + ch) * kExchangeFloats;
      if (wtid < 16) __stcg(mine + wtid, stat[wtid]);
      __threadfence();
      small_sync();
      if (wtid == 0) st_relaxed_u32(reinterpret_cast<uint32_t*>(mine + 16), A.stamp);
      bool ok = true;
      if (wtid < nch) {
        const uint32_t* theirs = reinterpret_cast<const uint32_t*>(
            p.att_xch + (static_cast<size_t>(rowg) * kMaxChunks + wtid) * kExchangeFloats + 16);
        uint32_t spins = 0;
        while (ld_relaxed_u32(theirs) != A.stamp) {
          if ((++spins & 255u) == 0 && give_up(cx, SITE_ATT_EXCHANGE, rowg)) {
            ok = false;
            break;
          }
        }
        __threadfence();
      }
      if (!small_ok(cx, ok)) return false;
      if (wtid < gs) {
        const float* all = p.att_xch + static_cast<size_t>(rowg) * kMaxChunks * kExchangeFloats;
        float m = -INFINITY;
        for (int c = 0; c < nch; ++c) m = fmaxf(m, __ldcg(all + c * kExchangeFloats + wtid));
        float s = 0.f;
        for (int c = 0; c < nch; ++c)
          s += __ldcg(all + c * kExchangeFloats + 8 + wtid) * expf(__ldcg(all + c * kExchangeFloats + wtid) - m);
        stat[wtid] = m;
        stat[8 + wtid] = s;
      }
      small_sync();
    }

    // --- probabilities (bf16, against the global max and sum) and value accumulation
    for (int g = 0; g < gs; ++g) {
      const float m = stat[g], denom = stat[8 + g];
      for (int i = wtid; i < cl; i += kSmallWorkers) sc[g * chunk + i] = bf16_round(expf(sc[g * chunk + i] - m) / denom);
    }
    small_sync();
    for (int g = 0; g < gs; ++g) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int base = j0 + warp * kpw; base < j1; base += pass * kU) {
        const bool first_batch = (base == j0 + warp * kpw);
        uint4 vv[kU];
#pragma unroll
        for (int u8 = 0; u8 < kU; ++u8) {
          const int j = base + u8 * pass + sub;
          vv[u8] = vu[u8];
          if (!first_batch) {
            vv[u8] = make_uint4(0, 0, 0, 0);
            if (j < j1 && j != newpos) vv[u8] = __ldcg(reinterpret_cast<const uint4*>(vbase + static_cast<long long>(j) * A.kv_ld) + dg);
          }
        }
#pragma unroll
        for (int u8 = 0; u8 < kU; ++u8) {
          const int j = base + u8 * pass + sub;
          if (j < j1) {
            if (j == newpos) vv[u8] = *reinterpret_cast<const uint4*>(vn + dg * 8);
            float vf[8];
            unpack8(vv[u8], vf);
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
      if (g > 0) small_sync();  // red is free (previous head consumed)
      if (sub == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) red[warp * 128 + dg * 8 + e] = acc[e];
      }
      small_sync();
      if (wtid < hd) {
        float o = red[wtid];
#pragma unroll
        for (int w8 = 1; w8 < kSmallWarps; ++w8) o += red[w8 * 128 + wtid];
        const int head = kvh * gs + g;
        if (nch == 1) {
          A.out[static_cast<long long>(b) * A.out_ld + head * hd + wtid] = __float2bfloat16_rn(o);
        } else {
          const size_t row = static_cast<size_t>(b) * p.q_heads + head;
          __stcg(p.att_part + (row * kMaxChunks + ch) * hd + wtid, o);
        }
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------------------
// consumers: whole-launch schedule (decode with the split-K phase table)

__device__ __forceinline__ uint4 small_norm_weight(const Ctx& cx, int gp, int wtid) {
  if (gp >= cx.p->n_gemm) return make_uint4(0, 0, 0, 0);
  const GemmPhase* ph = &cx.misc->phase[gp & 1];
  if (ph->bmode != B_NORM || wtid >= ph->k / 8) return make_uint4(0, 0, 0, 0);
  return __ldg(reinterpret_cast<const uint4*>(ph->normw) + wtid);
}

__device__ void small_worker_loop(const Ctx& cx, int wtid) {
  const KParams& p = *cx.p;
  SmallState st;
  st.head = 0; st.seq = 0; st.passed = 0;
  const int q_size = p.q_heads * p.head_dim, kv_size = p.kv_heads * p.head_dim;
  const int gs = p.q_heads / p.kv_heads;
  SmallAttn A;
  A.q = p.qkv; A.q_ld = p.qkv_ld;
  A.knew = p.qkv + q_size; A.vnew = A.knew + kv_size; A.new_ld = p.qkv_ld;
  A.out = p.attn; A.out_ld = q_size;
  A.kv_bstride = static_cast<long long>(p.capacity) * kv_size; A.kv_ld = kv_size;
  A.scale = p.att_scale;
  small_prefetch_phase(cx, 0, wtid);
  small_sync();
  uint4 wu = small_norm_weight(cx, 0, wtid);
  int step = 0;
#define MK_SMALL_STEP() do { if (p.debug_stop && ++step >= p.debug_stop) return; } while (0)
  // One projection phase: the next descriptor is fetched while this phase runs.
  bool ok = true;  // per warp; made block-uniform by every close()
  auto project = [&](int gp, int nch) {
    small_prefetch_phase(cx, gp + 1, wtid);
    ok = small_gemm_any(cx, gp, st, wtid, wu, nch) && ok;
  };
  // Close a phase: arrive, fetch what the next phase needs that no other CTA writes, wait.
  auto close = [&](int next_gp) -> bool {
    if (!ok) cx.misc->wabort = 1;
    small_arrive(cx, st, wtid);   // its bar.sync also publishes the prefetched descriptor to every consumer
    wu = small_norm_weight(cx, next_gp, wtid);
    return small_wait(cx, st, wtid);
  };
  for (int layer = 0; layer < p.layers; ++layer) {
    const int gp = layer * 4;
    project(gp, 1);                          // [residual update, RMSNorm] q, k, v (+bias)
    MK_SMALL_STEP();
    if (!close(gp + 1)) return;
    MK_SMALL_STEP();
    A.k = static_cast<bf16*>(p.kc[layer]); A.v = static_cast<bf16*>(p.vc[layer]);
    A.len = cx.misc->len_s[layer];
    A.stamp = p.att_epoch + static_cast<uint32_t>(layer) + 1u;
    const int nch = decode_chunks(A.len + 1, p.batch * p.kv_heads, cx.grid, gs);
    if (!small_attention(cx, A, wtid, nch)) return;       // RoPE, KV append, split-context attention
    trace_event(cx, wtid, EV_ATTENTION_DONE);
    MK_SMALL_STEP();
    if (!close(gp + 1)) return;
    if (cx.cta == 0 && wtid == 0) *p.len[layer] = A.len + 1;  // publish after the interval closes
    MK_SMALL_STEP();
    project(gp + 1, nch);                    // o_proj (fp32 K-slice partials)
    MK_SMALL_STEP();
    if (!close(gp + 2)) return;
    project(gp + 2, 1);                      // [residual update, RMSNorm] gate, up -> SiLU*up
    MK_SMALL_STEP();
    if (!close(gp + 3)) return;
    project(gp + 3, 1);                      // down (fp32 K-slice partials)
    MK_SMALL_STEP();
    if (!close(gp + 4)) return;
  }
#undef MK_SMALL_STEP
  project(p.layers * 4, 1);                               // [residual update, final RMSNorm] lm_head
}

// ---------------------------------------------------------------------------
// the kernel

__global__ void __launch_bounds__(kSmallThreads, 1) megakernel_small(const __grid_constant__ KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctx cx;
  cx.p = &p;
  cx.ctrl = p.ctrl;
  cx.smem_a = smem;
  cx.smem_b = smem + kRingBytes;
  cx.misc = reinterpret_cast<SmemMisc*>(cx.smem_b + kBBytes);
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
      if (id < 0 || id >= p.vocab || pos < 0 || pos >= p.max_positions) {
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
    if (tid == 0) {
      if (cx.cta == 0 && atomicCAS(&cx.ctrl->status, 0, bad) == 0) {
        cx.ctrl->where = SITE_PROLOGUE;
        cx.ctrl->cta = 0;
        cx.ctrl->detail = 0;
      }
      if (p.nbar > 0) atomicAdd(&cx.ctrl->barrier, static_cast<uint32_t>(p.nbar));  // keep the monotonic counter consistent
    }
  } else if (warp == 0) {
    if (tid == 0) producer_loop(cx);
  } else {
    small_worker_loop(cx, tid - 32);
  }
}

}  // namespace mk
