// Splash attention forward for head dims above 128 (q / k up to 256 columns, v / o up to 256),
// bf16, sm_100a.  The reference's kernel test draws (256, 256) and (192, 128) among its head dims
// (splash_attention_kernel_test.py:233-237) and its microbenchmarks quote both; the kernel it
// replaces is `flash_attention_kernel` (splash_attention_kernel.py:299-527), as for the 128-wide
// forward.
//
// A head dim above 128 is handled as up to two 128-column panels, each panel being the 128 x 128
// bf16 tile (two swizzled 64-column halves) the 128-wide kernels use, so that every MMA, TMA box and
// descriptor has the shape those kernels use:
//   S  = Q_a K_a^T + Q_b K_b^T            up to 16 K = 16 MMAs accumulating into one 128-column S
//   O[:, panel] (+)= P V[:, panel]        8 MMAs per V panel into that panel's 128 TMEM columns
// A panel's columns past the head dim arrive as zeros from TMA; a last panel of at most 64
// columns loads and multiplies one half only.
//
// One CTA works on ONE q tile (O alone takes up to 256 of the 512 TMEM columns):
//   TMEM  [0,128) S of even steps / P   [128,256) S of odd steps / P   [256,512) O
//   smem  Q panels 2 x 32 KiB, ring of 4 x 32 KiB panels (a step's K panels, then its V panels)
//   warps 0-7 softmax, warp 8 TMA producer, warp 9 MMA issuer (10, 11 idle)
// q k^T of step n+1 is issued before p v of step n, so the tensor core works on it while the
// softmax warps turn S(n) into P(n).  The softmax warps may rescale O only once p v of the
// previous step has completed (`pv_done`), which the lazy rescaling makes a rare wait.
// Softmax: the exponentials are bound by instruction issue, and one q tile gives one warpgroup
// only one warp per scheduler.  So two warpgroups share the tile: both own all 128 rows (a warp
// reaches the TMEM lanes of its index mod 4) and each takes 64 of the 128 key columns of a step;
// the two halves of a row's maximum (and, at the end, of its sum) meet through shared memory and an
// mbarrier (`mx_full`, bounded like every other wait), after which both warpgroups hold the same
// maximum and take the same rescaling decision.
// The schedule is the 128-wide forward's (rows = pairs of q tiles); a CTA follows the entries in
// which its own q tile is live.
#include <mutex>

#include "splash_common.cuh"
#include "splash_fwd_params.cuh"

namespace sb {

constexpr int kWideStages = 4;
constexpr int kWideThreads = 384;
constexpr int kWideHalf = kTile / 2;  // key columns of a step per softmax warpgroup
constexpr int kWideXchgBytes = 2 * 2 * kTile * 4;  // [step parity][column half][row] floats
constexpr int kWideSmemBytes = (2 + kWideStages) * kTileBytes + kWideXchgBytes + 1024 /*barriers*/ + 1024 /*alignment slack*/;

struct WideBarriers {
  uint64_t q_full;
  uint64_t kv_full[kWideStages];
  uint64_t kv_empty[kWideStages];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t pv_done;  // one phase per step: the p v MMAs of that step have completed
  uint64_t o_done;
  uint64_t mx_full;  // one phase per step (and one for the sums): all 8 softmax warps have published their half
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t early_exit;
};

// bytes TMA delivers for a panel holding `cols` real columns (1..128): one or two 64-column halves
__device__ __forceinline__ uint32_t panel_bytes(int cols) { return cols > 64 ? kTileBytes : kHalfBytes; }

template <bool kSoftCap>
__global__ void __launch_bounds__(kWideThreads, 1)
splash_fwd_wide_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;                    // 2 panels
  uint8_t* ring = smem + 2 * kTileBytes;     // kWideStages panels
  float* xchg = reinterpret_cast<float*>(smem + (2 + kWideStages) * kTileBytes);
  WideBarriers* bars = reinterpret_cast<WideBarriers*>(smem + (2 + kWideStages) * kTileBytes + kWideXchgBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // two CTAs per schedule row, one per q tile of the pair
  const CtaWork work = cta_work_at(blockIdx.x >> 1, p.row_order, p.n_rows, p.n_groups, p.chunk_groups, true);
  const int i = blockIdx.x & 1;
  const int q_tile = work.row * 2 + i;
  if (q_tile >= p.n_q_tiles) return;  // odd number of q tiles: the last row has one tile
  const int head = work.group % p.q_heads;
  const int batch = work.group / p.q_heads;
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int ebeg = p.row_ptr[work.row];
  const int eend = p.row_end ? p.row_end[(int64_t)batch * p.n_rows + work.row] : p.row_ptr[work.row + 1];
  const int4* entries = p.entries + (int64_t)batch * p.entries_per_batch;
  const int npk = (p.d_qk + kHeadDim - 1) / kHeadDim;  // panels of q / k
  const int npv = (p.d_v + kHeadDim - 1) / kHeadDim;   // panels of v / o

  if (threadIdx.x == 0) {
    bars->early_exit = *reinterpret_cast<volatile uint32_t*>(p.err);
    bars->abort_flag = 0;
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->pv_done, 1);
    mbar_init(&bars->o_done, 1);
    mbar_init(&bars->mx_full, 8);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1);
      mbar_init(&bars->p_full[b], 8);  // one arrival per softmax warp
    }
    for (int s = 0; s < kWideStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (bars->early_exit != 0) return;  // an earlier CTA already reported a fault

  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  AbortCtx ab{&bars->abort_flag, p.err};

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      uint32_t q_bytes = 0;
      for (int pp = 0; pp < npk; ++pp) q_bytes += panel_bytes(p.d_qk - pp * kHeadDim);
      mbar_arrive_expect_tx(&bars->q_full, q_bytes);
      for (int pp = 0; pp < npk; ++pp) {
        uint8_t* dst = q_smem + pp * kTileBytes;
        tma_load_4d(dst, &tm_q, &bars->q_full, pp * kHeadDim, q_tile * kTile, head, batch);
        if (p.d_qk - pp * kHeadDim > 64)
          tma_load_4d(dst + kHalfBytes, &tm_q, &bars->q_full, pp * kHeadDim + 64, q_tile * kTile, head, batch);
      }
      uint32_t it = 0;
      bool ok = true;
      for (int e = ebeg; e < eend && ok; ++e) {
        const int4 ent = entries[e];
        if (((ent.y >> (2 * i)) & 3) == 0) continue;
        for (int item = 0; item < npk + npv && ok; ++item, ++it) {
          const bool is_k = item < npk;
          const int pp = is_k ? item : item - npk;
          const int cols = (is_k ? p.d_qk : p.d_v) - pp * kHeadDim;
          const uint32_t s = it % kWideStages;
          ok = mbar_wait(&bars->kv_empty[s], ((it / kWideStages) & 1u) ^ 1u, ab, 0x900u + s);
          if (!ok) break;
          uint8_t* dst = ring + s * kTileBytes;
          const CUtensorMap* tm = is_k ? &tm_k : &tm_v;
          mbar_arrive_expect_tx(&bars->kv_full[s], panel_bytes(cols));
          tma_load_4d(dst, tm, &bars->kv_full[s], pp * kHeadDim, ent.x * kTile, kv_head, batch);
          if (cols > 64)
            tma_load_4d(dst + kHalfBytes, tm, &bars->kv_full[s], pp * kHeadDim + 64, ent.x * kTile, kv_head, batch);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(kTile, kTile, false, false);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t ring_addr = smem_u32(ring);
      bool ok = mbar_wait(&bars->q_full, 0, ab, 0xA00u);

      // The thread that issues the MMAs is alone in its warp: every instruction it spends between two
      // MMAs shows up as tensor-core idle time, so the loops below are unrolled over compile-time
      // offsets and everything that does not change from step to step is prepared here.
      SmemDesc q_desc[2];
      int nk_panel[2];
      uint32_t idesc_pv[2];
      for (int pp = 0; pp < 2; ++pp) {
        q_desc[pp] = make_smem_desc_sw128(q_addr + pp * kTileBytes, 16, 1024);
        const int cols = p.d_qk - pp * kHeadDim;
        nk_panel[pp] = cols >= kHeadDim ? 8 : (cols > 0 ? (cols + 15) / 16 : 0);
        idesc_pv[pp] = make_idesc_bf16(kTile, p.d_v - pp * kHeadDim > 64 ? kHeadDim : 64, false, true);
      }
      // S[buf] = sum over panels Q_pp K_pp^T; K panels sit in ring items it0 .. it0 + npk - 1
      auto issue_qk = [&](uint32_t buf, uint32_t it0) {
        const uint32_t d = tmem + buf * kTile;
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
          if (pp < npk) {
            const uint32_t slot = (it0 + pp) % kWideStages;
            const SmemDesc da = q_desc[pp];
            const SmemDesc db = make_smem_desc_sw128(ring_addr + slot * kTileBytes, 16, 1024);
            const int nk = nk_panel[pp];
            if (nk == 8) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
                umma_ss(d, desc_at(da, off), desc_at(db, off), idesc_qk, (pp > 0 || k > 0) ? 1u : 0u);
              }
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                if (k < nk) {
                  const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
                  umma_ss(d, desc_at(da, off), desc_at(db, off), idesc_qk, (pp > 0 || k > 0) ? 1u : 0u);
                }
              }
            }
          }
        }
        tc_commit(&bars->s_full[buf]);
        tc_commit(&bars->kv_empty[it0 % kWideStages]);
        if (npk > 1) tc_commit(&bars->kv_empty[(it0 + 1) % kWideStages]);
      };
      // O[:, panel] (+)= P[buf] V_panel; V panels sit in ring items it0 .. it0 + npv - 1
      auto issue_pv = [&](uint32_t buf, uint32_t it0, bool acc) {
        const uint32_t a = tmem + buf * kTile;
#pragma unroll
        for (int vp = 0; vp < 2; ++vp) {
          if (vp < npv) {
            const uint32_t slot = (it0 + vp) % kWideStages;
            const SmemDesc db = make_smem_desc_sw128(ring_addr + slot * kTileBytes, kHalfBytes, 1024);
            const uint32_t d = tmem + 2 * kTile + vp * kHeadDim;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_ts(d, a + k * 8, desc_at(db, k * 2048), idesc_pv[vp], (acc || k > 0) ? 1u : 0u);
          }
        }
        tc_commit(&bars->kv_empty[it0 % kWideStages]);
        if (npv > 1) tc_commit(&bars->kv_empty[(it0 + 1) % kWideStages]);
        tc_commit(&bars->pv_done);
      };
      auto wait_items = [&](uint32_t it0, int count, uint32_t tag) {
        bool good = true;
        for (int j = 0; j < count && good; ++j) {
          const uint32_t itj = it0 + j;
          good = mbar_wait(&bars->kv_full[itj % kWideStages], (itj / kWideStages) & 1u, ab, tag + j);
        }
        return good;
      };
      auto next_live = [&](int e) {
        while (e < eend && ((entries[e].y >> (2 * i)) & 3) == 0) ++e;
        return e;
      };

      int e = next_live(ebeg);
      uint32_t it = 0, n = 0;
      uint32_t v_it = 0;  // ring item of the first V panel of the step whose p v comes next
      if (e < eend && ok) {
        ok = wait_items(it, npk, 0xA10u);
        if (ok) {
          mma_issue_fence();
          issue_qk(0, it);
          v_it = it + npk;
          it += npk + npv;
        }
        while (ok) {
          const int e_next = next_live(e + 1);
          const bool has_next = e_next < eend;
          uint32_t v_it_next = 0;
          if (has_next) {
            ok = wait_items(it, npk, 0xA20u);
            if (!ok) break;
            mma_issue_fence();
            issue_qk((n + 1) & 1u, it);
            v_it_next = it + npk;
            it += npk + npv;
          }
          ok = mbar_wait(&bars->p_full[n & 1u], (n >> 1) & 1u, ab, 0xA30u + (n & 1u));
          if (ok) ok = wait_items(v_it, npv, 0xA40u);
          if (!ok) break;
          mma_issue_fence();
          issue_pv(n & 1u, v_it, n > 0);
          if (!has_next) break;
          v_it = v_it_next;
          e = e_next;
          ++n;
        }
      }
      tc_commit(&bars->o_done);
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax warps
    const int half = warp >> 2;        // which 64 key columns of a step this warpgroup takes
    const int wq = warp & 3;           // TMEM lane quarter this warp may touch
    const int r = wq * 32 + lane;      // row within the tile
    const int c0 = half * kWideHalf;   // first key column of this half
    const int q_row = q_tile * kTile + r;
    const int qi = p.q_sequence ? p.q_sequence[q_row] : q_row;
    const RowInterval iv = mask_fn_interval(p.fn, qi);
    const bool has_seg = p.q_seg != nullptr;
    const int q_seg = has_seg ? p.q_seg[(int64_t)batch * p.q_len + q_row] : 0;
    const int32_t* kv_seg_row = has_seg ? p.kv_seg + (int64_t)batch * p.kv_len : nullptr;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const uint32_t t_o = tmem + lane_addr + 2 * kTile;
    const float c = fmaxf(kSoftCap ? p.soft_cap * kLog2e : p.scale_log2, kMinScaleLog2);  // score -> log2 units
    // 32-column groups of O that hold real columns, shared out between the two warpgroups
    const int o_groups = (p.d_v + 31) / 32;
    const int og_begin = half == 0 ? 0 : (o_groups + 1) / 2;
    const int og_end = half == 0 ? (o_groups + 1) / 2 : o_groups;

    float m_used = -INFINITY;  // scaled (log2) units
    float m_true = kMaskedLogit;
    float l = 0.f;             // this half's share of the row sum (a sink is counted by half 0)
    const bool fixed_max = p.max_logit_value != nullptr;
    float sink2 = -INFINITY;  // sink logit in log2 units
    if (p.sinks != nullptr) sink2 = p.sinks[head] * kLog2e;
    if (fixed_max) {
      m_used = p.max_logit_value[head] * kLog2e;
      if (p.sinks != nullptr && half == 0) l = ex2(sink2 - m_used);
    } else if (p.sinks != nullptr) {
      m_used = sink2;
      if (half == 0) l = 1.f;
    }
    uint32_t n = 0;
    bool ok = true;

    for (int e = ebeg; e < eend; ++e) {
      const int4 ent = entries[e];
      const int st = (ent.y >> (2 * i)) & 3;
      if (st == 0) continue;
      const uint32_t buf = n & 1u;
      const uint32_t t_s = tmem + lane_addr + buf * kTile;
      ok = mbar_wait(&bars->s_full[buf], (n >> 1) & 1u, ab, 0xB00u + buf);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();

      float s[kWideHalf];
      {
        uint32_t v0[32], v1[32];
        tmem_ld32(t_s + c0, v0);
        tmem_ld32(t_s + c0 + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          s[j] = __uint_as_float(v0[j]);
          s[32 + j] = __uint_as_float(v1[j]);
        }
      }
      if constexpr (kSoftCap) {
#pragma unroll
        for (int j = 0; j < kWideHalf; ++j) s[j] = tanh_ex2(s[j] * p.softcap_a);
      }
      const int kv0 = ent.x * kTile + c0;  // first key of this half
      if (st == 1) {
        if (p.fn.kind != SPLASH_MASK_TABLE) {
          const int lo_rel = iv.lo <= kv0 ? 0 : iv.lo - kv0;
          const int hi_rel = iv.hi >= kv0 + (kWideHalf - 1) ? kWideHalf - 1 : iv.hi - kv0;
#pragma unroll
          for (int j = 0; j < kWideHalf; ++j)
            if (j < lo_rel || j > hi_rel) s[j] = kMaskedLogit;
        } else {
          const int pid = i == 0 ? ent.z : ent.w;
          const int8_t* mrow = p.pmb + ((int64_t)pid * p.pm_bq + (q_row % p.pm_bq)) * p.pm_bkv + (kv0 % p.pm_bkv);
          const int4* m4 = reinterpret_cast<const int4*>(mrow);
#pragma unroll
          for (int g = 0; g < kWideHalf / 16; ++g) {
            const int4 mv = __ldg(m4 + g);
            const uint32_t w[4] = {(uint32_t)mv.x, (uint32_t)mv.y, (uint32_t)mv.z, (uint32_t)mv.w};
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (((w[j >> 2] >> ((j & 3) * 8)) & 0xffu) == 0u) s[g * 16 + j] = kMaskedLogit;
          }
        }
      }
      if (has_seg && !((ent.y >> (4 + i)) & 1)) {  // (bit set: the whole tile lies inside one segment)
        const int4* sg4 = reinterpret_cast<const int4*>(kv_seg_row + kv0);
#pragma unroll
        for (int g = 0; g < kWideHalf / 4; ++g) {
          const int4 sv = __ldg(sg4 + g);
          if (sv.x != q_seg) s[g * 4 + 0] = kMaskedLogit;
          if (sv.y != q_seg) s[g * 4 + 1] = kMaskedLogit;
          if (sv.z != q_seg) s[g * 4 + 2] = kMaskedLogit;
          if (sv.w != q_seg) s[g * 4 + 3] = kMaskedLogit;
        }
      }

      float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
      float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
      for (int j = 12; j < kWideHalf - 4; j += 8) {
        mx0 = max3(mx0, s[j], s[j + 1]);
        mx1 = max3(mx1, s[j + 2], s[j + 3]);
        mx2 = max3(mx2, s[j + 4], s[j + 5]);
        mx3 = max3(mx3, s[j + 6], s[j + 7]);
      }
      mx0 = max3(mx0, s[kWideHalf - 4], s[kWideHalf - 3]);
      mx1 = max3(mx1, s[kWideHalf - 2], s[kWideHalf - 1]);
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      // the other half's maximum of the same row
      float* slot = xchg + (n & 1u) * (2 * kTile);
      slot[half * kTile + r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->mx_full);
      ok = mbar_wait(&bars->mx_full, n & 1u, ab, 0xB30u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      mx = fmaxf(mx, slot[(half ^ 1) * kTile + r]);

      const float m_new = fmaxf(mx * c, kLogitFloor);
      m_true = fmaxf(m_true, mx);
      const bool need = !fixed_max && m_new > m_used + kRescaleThreshold;
      if (__any_sync(0xffffffffu, need)) {
        const float m_next = fmaxf(m_used, m_new);
        const float alpha = ex2(m_used - m_next);
        l *= alpha;
        if (n > 0) {
          // O still receives p v of the previous step: wait for it before touching O
          ok = mbar_wait(&bars->pv_done, (n - 1) & 1u, ab, 0xB10u);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          uint32_t v[32];
          for (int g = og_begin; g < og_end; ++g) {
            tmem_ld32(t_o + g * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
            tmem_st32(t_o + g * 32, v);
          }
        }
        m_used = m_next;
      }

      const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_used, -m_used);
      float2 lsa = make_float2(0.f, 0.f), lsb = make_float2(0.f, 0.f);
#pragma unroll
      for (int g = 0; g < kWideHalf / 32; ++g) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float2 xa = __ffma2_rn(make_float2(s[g * 32 + 2 * j], s[g * 32 + 2 * j + 1]), c2, nm2);
          const float2 xb = __ffma2_rn(make_float2(s[g * 32 + 2 * j + 2], s[g * 32 + 2 * j + 3]), c2, nm2);
          const float2 pa = make_float2(ex2(xa.x), ex2(xa.y));
          const float2 pb = make_float2(ex2(xb.x), ex2(xb.y));
          lsa = __fadd2_rn(lsa, pa);
          lsb = __fadd2_rn(lsb, pb);
          pk[j] = pack_bf16(pa.x, pa.y);
          pk[j + 1] = pack_bf16(pb.x, pb.y);
        }
        tmem_st16(t_s + c0 / 2 + g * 16, pk);  // P: two bf16 per 32-bit column
      }
      l += (lsa.x + lsb.x) + (lsa.y + lsb.y);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[buf]);
      ++n;
    }

    // ---- the row sums of the two halves meet (one more phase of the exchange barrier)
    if (ok) {
      float* slot = xchg + (n & 1u) * (2 * kTile);
      slot[half * kTile + r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->mx_full);
      ok = mbar_wait(&bars->mx_full, n & 1u, ab, 0xB40u);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) l += slot[(half ^ 1) * kTile + r];
    }
    // ---- epilogue: O / l -> bf16 (each warpgroup its share of the columns), logsumexp, max_logits
    if (ok) {
      ok = mbar_wait(&bars->o_done, 0, ab, 0xB20u);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* orow = p.o + (int64_t)batch * p.o_sb + (int64_t)head * p.o_sh + (int64_t)q_row * p.o_ss;
      uint4* o4 = reinterpret_cast<uint4*>(orow);
      const bool live = l > 0.f;  // a row that met a live key, or has a sink
      const float inv = live ? 1.0f / l : 0.f;
      for (int g = og_begin; g < og_end; ++g) {
        uint32_t v[32];
        if (n > 0) {
          tmem_ld32(t_o + g * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(v[8 * j + 0]) * inv, __uint_as_float(v[8 * j + 1]) * inv);
          w.y = pack_bf16(__uint_as_float(v[8 * j + 2]) * inv, __uint_as_float(v[8 * j + 3]) * inv);
          w.z = pack_bf16(__uint_as_float(v[8 * j + 4]) * inv, __uint_as_float(v[8 * j + 5]) * inv);
          w.w = pack_bf16(__uint_as_float(v[8 * j + 6]) * inv, __uint_as_float(v[8 * j + 7]) * inv);
          if ((g * 4 + j) * 8 < p.d_v) o4[g * 4 + j] = w;
        }
      }
      if (half == 0) {
        const int64_t stat = ((int64_t)batch * p.q_heads + head) * p.q_len + q_row;
        if (p.lse) p.lse[stat] = live ? (m_used + log2f(l)) * kLn2 : p.mask_value;
        if (p.maxl) {
          float mv = m_true * (kSoftCap ? p.soft_cap : p.scale);
          if (p.sinks != nullptr) mv = fmaxf(mv, sink2 * kLn2);
          if (fixed_max) mv = m_used * kLn2;
          p.maxl[stat] = live ? mv : p.mask_value;
        }
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

int launch_fwd_wide(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                    const FwdParams& p, bool soft_cap, cudaStream_t stream) {
  const int64_t blocks = 2ll * p.n_rows * p.n_groups;
  if (blocks > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;
  const void* fn = soft_cap ? (const void*)splash_fwd_wide_kernel<true> : (const void*)splash_fwd_wide_kernel<false>;
  {
    static std::mutex attr_mu;
    static bool attr_done[64][2] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SPLASH_ERR_CUDA;
    std::lock_guard<std::mutex> lock(attr_mu);
    if (!attr_done[dev][soft_cap ? 1 : 0]) {
      if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kWideSmemBytes) != cudaSuccess)
        return SPLASH_ERR_CUDA;
      attr_done[dev][soft_cap ? 1 : 0] = true;
    }
  }
  dim3 grid((unsigned)blocks, 1u, 1u);
  if (soft_cap)
    splash_fwd_wide_kernel<true><<<grid, kWideThreads, kWideSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
  else
    splash_fwd_wide_kernel<false><<<grid, kWideThreads, kWideSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}

}  // namespace sb
