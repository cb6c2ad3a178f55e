// Splash attention backward for head dims above 128 (q / k up to 256 columns, v / o up to 256),
// bf16, sm_100a: dq, dk and dv as three passes of one kernel.  Same arithmetic as the 128-wide
// backward (reference: splash_attention_kernel.py:1234-1459, base.py:115-173): P = exp(S - lse),
// dS = P * (dP - di), dq = dS k, dk = dS^T q, dv = P^T do, the q heads of a kv head summed inside
// one CTA (no atomics, bitwise repeatable).
//
// A head dim above 128 is two 128-column panels, each the 128 x 128 bf16 tile of the other
// kernels (see splash_fwd_wide_sm100.cu), so every TMA box, descriptor and MMA has a shape those
// kernels use.  With 256 output columns in TMEM there is room for one S and one dP beside them,
// and dk and dv together do not fit at all, so the work is cut into three passes that each hold
//   TMEM  [0,128) S (then the packed bf16 P or dS, the A operand of the output MMA)
//         [128,256) dP            [256,512) the pass's output, up to 256 columns
// pass   stationary (loaded once)   streamed per step: held / passing     output
//  dq    Q panels, dO panels        K panels / V panels                   dq += dS k
//  dk    K panels, V panels         Q panels / dO panels                  dk += dS^T q   (over the q-head group)
//  dv    K panels                   dO panels / Q panels                  dv += P^T do   (over the q-head group)
// "held" panels feed the output MMA, after the element-wise phase, so they stay for the whole step;
// "passing" panels go one after the other (through one slot; two in the dv pass) into an MMA that
// accumulates over them (dP over the V / dO panels; in the dv pass S over the Q panels).  S of the
// dq / dk passes multiplies the stationary panels with the held ones.  In the dk / dv passes the
// tile is transposed (threads own kv rows, columns are query rows), so logsumexp and di come per
// column and the mask function is evaluated per element, as in the 128-wide dkv kernel.
// Shared memory: seven panels of 32 KiB — dq / dk: 4 stationary + 2 held + 1 passing; dv (no second
// stationary operand): 2 stationary + a ring of 3 held + 2 passing.  A step's first passing panel is
// loaded while the previous step is still in its element-wise phase (dq / dk with two passing
// panels: the first half of dP is issued ahead of S, whose held panels arrive later; dv: both Q
// panels and one dO panel of the next step, and S^T alternates between two TMEM buffers — the dP
// columns are free there — so S^T(n+1) runs under the element-wise phase of step n).  The held
// panels of dq / dk are loaded only once the previous output MMAs have released them.  Built for
// coverage of the reference's head dims rather than tuned: S is computed in all three passes.
#include <mutex>

#include "splash_common.cuh"
#include "splash_bwd_params.cuh"

namespace sb {

enum WidePass { kWideDq = 0, kWideDk = 1, kWideDv = 2 };

constexpr int kWideBwdSmemBytes = 7 * kTileBytes + 1024 /*barriers*/ + 1024 /*alignment slack*/;

struct WideBwdBarriers {
  uint64_t stat_full;
  uint64_t held_full[3];
  uint64_t held_empty[3];
  uint64_t pass_full[2];
  uint64_t pass_empty[2];
  uint64_t s_full[2];   // dv pass: S alternates between two TMEM buffers; dq / dk: [0] only
  uint64_t dp_full;
  uint64_t ds_full[2];  // P (dv pass, per S buffer) or dS written back; one arrival per compute warp
  uint64_t acc_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t early_exit;
};

// One 128-row panel with `cols` real columns (1..128) starting at column x0: one or two boxes.
__device__ __forceinline__ void load_panel(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int cols, int x0,
                                           int row0, int head, int batch) {
  tma_load_4d(dst, tm, bar, x0, row0, head, batch);
  if (cols > 64) tma_load_4d(dst + kHalfBytes, tm, bar, x0 + 64, row0, head, batch);
}
__device__ __forceinline__ uint32_t wide_panel_bytes(int cols) { return cols > 64 ? kTileBytes : kHalfBytes; }
__device__ __forceinline__ int panel_cols(int d, int pp) { return d - pp * kHeadDim < kHeadDim ? d - pp * kHeadDim : kHeadDim; }

template <int kPass, bool kSoftCap>
__global__ void __launch_bounds__(kBwdThreads, 1)
splash_bwd_wide_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* a1_smem = smem;                      // 2 panels: Q (dq pass) or K
  uint8_t* a2_smem = smem + 2 * kTileBytes;     // 2 panels: dO (dq pass) or V; unused in the dv pass
  // held panels: a ring of two slots (a step's panels), or of three in the dv pass, which has the
  // panel behind them to spare: a panel of the next step's dO is then loaded under this step
  constexpr uint32_t kHeldSlots = kPass == kWideDv ? 3u : 2u;
  uint8_t* held_smem = smem + 4 * kTileBytes;
  // passing panels: one slot behind the held ones; the dv pass has no second stationary operand and
  // takes that operand's two panels as two slots instead, so a whole step's Q panels are prefetched
  constexpr uint32_t kPassSlots = kPass == kWideDv ? 2u : 1u;
  uint8_t* pass_smem = kPass == kWideDv ? a2_smem : smem + 6 * kTileBytes;
  WideBwdBarriers* bars = reinterpret_cast<WideBwdBarriers*>(smem + 7 * kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const CtaWork work = cta_work(p.row_order, p.n_rows, p.n_groups, p.chunk_groups, true);
  const int tile = work.row;  // q tile (dq pass) or kv tile
  const int group = p.q_heads / p.kv_heads;
  // dq pass: a CTA belongs to one (batch, q head); dk / dv: to one (batch, kv head) and walks its q heads
  const int heads_here = kPass == kWideDq ? 1 : group;
  const int batch = work.group / (kPass == kWideDq ? p.q_heads : p.kv_heads);
  const int own_head = work.group % (kPass == kWideDq ? p.q_heads : p.kv_heads);
  const int kv_head = kPass == kWideDq ? own_head / group : own_head;
  const int ebeg = p.row_ptr[tile];
  const int eend = p.row_end ? p.row_end[(int64_t)batch * p.n_rows + tile] : p.row_ptr[tile + 1];
  const int4* entries = p.entries + (int64_t)batch * p.entries_per_batch;
  const int n_ent = eend - ebeg;
  const int n_steps = n_ent * heads_here;
  const int npk = (p.d_qk + kHeadDim - 1) / kHeadDim;
  const int npv = (p.d_v + kHeadDim - 1) / kHeadDim;
  const int n_held = kPass == kWideDv ? npv : npk;  // panels that feed the output MMA
  const int n_pass = kPass == kWideDv ? npk : npv;  // panels that go through the single slot
  const int d_held = kPass == kWideDv ? p.d_v : p.d_qk;
  const int d_pass = kPass == kWideDv ? p.d_qk : p.d_v;

  if (threadIdx.x == 0) {
    bars->early_exit = *reinterpret_cast<volatile uint32_t*>(p.err);
    bars->abort_flag = 0;
    mbar_init(&bars->stat_full, 1);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bars->held_full[i], 1);
      mbar_init(&bars->held_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->pass_full[i], 1);
      mbar_init(&bars->pass_empty[i], 1);
    }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->ds_full[0], 8);
    mbar_init(&bars->ds_full[1], 8);
    mbar_init(&bars->acc_done, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (bars->early_exit != 0) return;
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  AbortCtx ab{&bars->abort_flag, p.err};
  const uint32_t t_s = tmem, t_dp = tmem + kTile, t_out = tmem + 2 * kTile;

  if (warp >= 8) {
   setmaxnreg_dec<kIssueRegs>();
   if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_steps > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const CUtensorMap* tm_a1 = kPass == kWideDq ? &tm_q : &tm_k;
      const CUtensorMap* tm_a2 = kPass == kWideDq ? &tm_do : &tm_v;
      const CUtensorMap* tm_held = kPass == kWideDq ? &tm_k : (kPass == kWideDk ? &tm_q : &tm_do);
      const CUtensorMap* tm_pass = kPass == kWideDq ? &tm_v : (kPass == kWideDk ? &tm_do : &tm_q);
      uint32_t stat_bytes = 0;
      for (int pp = 0; pp < npk; ++pp) stat_bytes += wide_panel_bytes(panel_cols(p.d_qk, pp));
      if (kPass != kWideDv)
        for (int vp = 0; vp < npv; ++vp) stat_bytes += wide_panel_bytes(panel_cols(p.d_v, vp));
      mbar_arrive_expect_tx(&bars->stat_full, stat_bytes);
      for (int pp = 0; pp < npk; ++pp)
        load_panel(a1_smem + pp * kTileBytes, tm_a1, &bars->stat_full, panel_cols(p.d_qk, pp), pp * kHeadDim,
                   tile * kTile, own_head, batch);
      if (kPass != kWideDv)
        for (int vp = 0; vp < npv; ++vp)
          load_panel(a2_smem + vp * kTileBytes, tm_a2, &bars->stat_full, panel_cols(p.d_v, vp), vp * kHeadDim,
                     tile * kTile, own_head, batch);
      uint32_t n = 0;
      bool ok = true;
      auto load_held = [&](int col, int head) {
        for (int hp = 0; hp < n_held && ok; ++hp) {
          const uint32_t it = n * (uint32_t)n_held + hp;
          const uint32_t slot = kHeldSlots == 2 ? (uint32_t)hp : it % kHeldSlots;
          const uint32_t phase = kHeldSlots == 2 ? (n & 1u) : ((it / kHeldSlots) & 1u);
          ok = mbar_wait(&bars->held_empty[slot], phase ^ 1u, ab, 0xC00u + slot);
          if (!ok) break;
          const int cols = panel_cols(d_held, hp);
          mbar_arrive_expect_tx(&bars->held_full[slot], wide_panel_bytes(cols));
          load_panel(held_smem + slot * kTileBytes, tm_held, &bars->held_full[slot], cols, hp * kHeadDim, col * kTile,
                     head, batch);
        }
      };
      auto load_pass = [&](int col, int head, int first, int last) {  // passing panels first .. last - 1
        for (int pp = first; pp < last && ok; ++pp) {
          const uint32_t it = n * (uint32_t)n_pass + pp, slot = it % kPassSlots;
          ok = mbar_wait(&bars->pass_empty[slot], ((it / kPassSlots) & 1u) ^ 1u, ab, 0xC10u + slot);
          if (!ok) break;
          const int cols = panel_cols(d_pass, pp);
          mbar_arrive_expect_tx(&bars->pass_full[slot], wide_panel_bytes(cols));
          load_panel(pass_smem + slot * kTileBytes, tm_pass, &bars->pass_full[slot], cols, pp * kHeadDim, col * kTile,
                     head, batch);
        }
      };
      for (int g = 0; g < heads_here && ok; ++g) {
        // streamed tiles: K / V of the kv head (dq pass) or Q / dO of q head g of the group
        const int head = kPass == kWideDq ? kv_head : kv_head * group + g;
        for (int e = ebeg; e < eend && ok; ++e, ++n) {
          const int col = entries[e].x;
          // In the order the issuer takes them (the slots free up in that order too).  dq / dk: the
          // first passing panel was free since the previous step's dP, so it is in flight long before
          // the held panels, which wait for the previous step's output MMAs.
          if (kPass == kWideDv) {
            load_pass(col, head, 0, n_pass);
            load_held(col, head);
          } else {
            load_pass(col, head, 0, 1);
            load_held(col, head);
            load_pass(col, head, 1, n_pass);
          }
        }
      }
    }
   } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(kTile, kTile, false, false);
      const uint32_t a1_addr = smem_u32(a1_smem), a2_addr = smem_u32(a2_smem);
      const uint32_t held_addr = smem_u32(held_smem), pass_addr = smem_u32(pass_smem);
      // D (+)= A B^T, both K-major, over the `cols` real columns of one panel pair
      auto ss_kmajor = [&](uint32_t d, uint32_t a0, uint32_t b0, int cols, bool acc) {
        const SmemDesc da = make_smem_desc_sw128(a0, 16, 1024), db = make_smem_desc_sw128(b0, 16, 1024);
        const int nk = cols >= kHeadDim ? 8 : (cols + 15) / 16;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (nk != 8 && k >= nk) break;
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          umma_ss(d, desc_at(da, off), desc_at(db, off), idesc_kk, (acc || k > 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(&bars->stat_full, 0, ab, 0xD00u);
      // The dv pass has no dP, so its TMEM columns serve as a second S buffer: S^T of step n+1 is
      // issued (on the prefetched Q panels) before the output MMAs of step n, and runs while the
      // compute warps turn S^T(n) into P^T(n).  s_buf(n): S buffer of step n; its barriers complete
      // once per use.
      // slot and barrier phase of held panel hp of step n.  With two slots and a step that may hold
      // two panels the ring degenerates to slot = hp, once per step (kept free of arithmetic: the
      // issuing thread is alone in its warp and pays for every instruction between two MMAs).
      auto held_slot = [&](uint32_t n, int hp) -> uint32_t {
        if (kHeldSlots == 2) return (uint32_t)hp;
        return (n * (uint32_t)n_held + hp) % kHeldSlots;
      };
      auto held_phase = [&](uint32_t n, int hp) -> uint32_t {
        if (kHeldSlots == 2) return n & 1u;
        return ((n * (uint32_t)n_held + hp) / kHeldSlots) & 1u;
      };
      auto wait_held = [&](uint32_t n) {
        bool good = true;
        for (int hp = 0; hp < n_held && good; ++hp)
          good = mbar_wait(&bars->held_full[held_slot(n, hp)], held_phase(n, hp), ab, 0xD10u + hp);
        return good;
      };
      auto s_buf = [&](uint32_t n) { return kPass == kWideDv ? (n & 1u) : 0u; };
      auto s_use = [&](uint32_t n) { return kPass == kWideDv ? (n >> 1) : n; };
      // passing panel pp of step n into an accumulating MMA with stationary panel a0 + pp
      auto mma_passing = [&](uint32_t n, uint32_t d, uint32_t a0, int dim, int pp) {
          const uint32_t it = n * (uint32_t)n_pass + pp, slot = it % kPassSlots;
          if (!mbar_wait(&bars->pass_full[slot], (it / kPassSlots) & 1u, ab, 0xD20u + slot)) return false;
          mma_issue_fence();
          ss_kmajor(d, a0 + pp * kTileBytes, pass_addr + slot * kTileBytes, panel_cols(dim, pp), pp > 0);
          tc_commit(&bars->pass_empty[slot]);
          return true;
      };
      auto dv_scores = [&](uint32_t n) {  // S^T(n) = sum over panels k (passing q)^T
        bool good = true;
        for (int pp = 0; pp < npk && good; ++pp) good = mma_passing(n, t_s + s_buf(n) * kTile, a1_addr, p.d_qk, pp);
        if (good) tc_commit(&bars->s_full[s_buf(n)]);
        return good;
      };
      if (kPass == kWideDv && ok) ok = dv_scores(0);
      for (uint32_t n = 0; n < (uint32_t)n_steps && ok; ++n) {
        if (kPass != kWideDv) {
          // dP = sum over panels (stationary do or v) (passing v or do)^T: its first panel was loaded
          // during the previous step; the dP columns are free since that step's ds_full
          // (with two passing panels the first goes ahead of S, so that the second can load under S;
          // with one, S goes first and the element-wise phase starts on it while dP runs)
          if (npv > 1) ok = mma_passing(n, t_dp, a2_addr, p.d_v, 0);
          if (!ok) break;
          ok = wait_held(n);
          if (!ok) break;
          mma_issue_fence();
          for (int pp = 0; pp < npk; ++pp)  // S = sum over panels (stationary q or k) (held k or q)^T
            ss_kmajor(t_s, a1_addr + pp * kTileBytes, held_addr + held_slot(n, pp) * kTileBytes, panel_cols(p.d_qk, pp), pp > 0);
          tc_commit(&bars->s_full[0]);
          for (int vp = npv > 1 ? 1 : 0; vp < npv && ok; ++vp) ok = mma_passing(n, t_dp, a2_addr, p.d_v, vp);
          if (!ok) break;
          tc_commit(&bars->dp_full);
        } else {
          if (n + 1 < (uint32_t)n_steps) ok = dv_scores(n + 1);
          ok = ok && wait_held(n);
          if (!ok) break;
        }
        ok = mbar_wait(&bars->ds_full[s_buf(n)], s_use(n) & 1u, ab, 0xD30u);
        if (!ok) break;
        mma_issue_fence();
        // out[:, panel] (+)= (packed P or dS in the S columns) (held panel read MN-major)
        for (int hp = 0; hp < n_held; ++hp) {
          const uint32_t idesc_mn = make_idesc_bf16(kTile, panel_cols(d_held, hp) > 64 ? kHeadDim : 64, false, true);
          const SmemDesc db = make_smem_desc_sw128(held_addr + held_slot(n, hp) * kTileBytes, kHalfBytes, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_ts(t_out + hp * kHeadDim, t_s + s_buf(n) * kTile + packed_a_col(k), desc_at(db, k * 2048), idesc_mn,
                    (n > 0 || k > 0) ? 1u : 0u);
          tc_commit(&bars->held_empty[held_slot(n, hp)]);
        }
      }
      tc_commit(&bars->acc_done);
    }
   }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    setmaxnreg_inc<kComputeRegs>();
    const int w = warp >> 2;       // which 64 columns of the step's tile this warpgroup takes
    const int wq = warp & 3;       // TMEM lane quarter
    const int r = wq * 32 + lane;  // row within the tile: a q row (dq pass) or a kv row
    const int row = tile * kTile + r;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c = kSoftCap ? p.soft_cap * kLog2e : p.scale_log2;
    const bool has_seg = p.q_seg != nullptr;
    // dq pass: everything per row is fixed for the CTA
    int own_seg = 0;
    RowInterval iv{INT32_MIN, INT32_MAX};
    float row_nlse2 = 0.f, row_ndelta = 0.f;
    if (kPass == kWideDq) {
      const int qi = p.q_sequence ? p.q_sequence[row] : row;
      iv = mask_fn_interval(p.fn, qi);
      own_seg = has_seg ? p.q_seg[(int64_t)batch * p.q_len + row] : 0;
      const int64_t stat = ((int64_t)batch * p.q_heads + own_head) * p.q_len + row;
      row_nlse2 = p.nlse2[stat];
      row_ndelta = p.delta[stat];
    } else {
      own_seg = has_seg ? p.kv_seg[(int64_t)batch * p.kv_len + row] : 0;
    }
    const int32_t* other_seg = has_seg ? (kPass == kWideDq ? p.kv_seg + (int64_t)batch * p.kv_len
                                                             : p.q_seg + (int64_t)batch * p.q_len)
                                       : nullptr;
    bool ok = true;
    uint32_t n = 0;

    for (int g = 0; g < heads_here && ok; ++g) {
      const int head = kPass == kWideDq ? own_head : kv_head * group + g;
      const int64_t stat_base = ((int64_t)batch * p.q_heads + head) * p.q_len;
      for (int e = ebeg; e < eend && ok; ++e, ++n) {
        const int4 ent = entries[e];
        const int st = ent.y & 3;
        const int c0 = ent.x * kTile + w * 64;  // first column: a key (dq pass) or a query row
        const uint32_t sb = kPass == kWideDv ? (n & 1u) : 0u;               // S buffer of this step
        const uint32_t s_phase = (kPass == kWideDv ? (n >> 1) : n) & 1u;   // and how often it was used
        const uint32_t t_sn = t_s + sb * kTile;
        ok = mbar_wait(&bars->s_full[sb], s_phase, ab, 0xE00u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float pr[64];
        {
          uint32_t v0[32], v1[32];
          tmem_ld32(t_sn + lane_addr + w * 64, v0);
          tmem_ld32(t_sn + lane_addr + w * 64 + 32, v1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            pr[j] = __uint_as_float(v0[j]);
            pr[32 + j] = __uint_as_float(v1[j]);
          }
        }
        if constexpr (kSoftCap) {  // pr <- tanh(scale * s / cap), capped before it is masked
#pragma unroll
          for (int j = 0; j < 64; ++j) pr[j] = tanh_ex2(pr[j] * p.softcap_a);
        }
        if (st == 1) {
          if (p.fn.kind != SPLASH_MASK_TABLE) {
            if (kPass == kWideDq) {
              const int lo_rel = iv.lo <= c0 ? 0 : iv.lo - c0;
              const int hi_rel = iv.hi >= c0 + 63 ? 63 : iv.hi - c0;
#pragma unroll
              for (int j = 0; j < 64; ++j)
                if (j < lo_rel || j > hi_rel) pr[j] = kMaskedLogit;
            } else {
#pragma unroll
              for (int j = 0; j < 64; ++j) {
                const int qi = p.q_sequence ? __ldg(p.q_sequence + c0 + j) : c0 + j;
                const RowInterval ivj = mask_fn_interval(p.fn, qi);
                if (row < ivj.lo || row > ivj.hi) pr[j] = kMaskedLogit;
              }
            }
          } else {
            // partial blocks: [id][q][kv] for the dq pass, stored transposed ([id][kv][q]) for dk / dv
            const int8_t* mrow =
                kPass == kWideDq
                    ? p.pmb + ((int64_t)ent.z * p.pm_bq + (row % p.pm_bq)) * p.pm_bkv + (c0 % p.pm_bkv)
                    : p.pmb + ((int64_t)ent.z * p.pm_bkv + (row % p.pm_bkv)) * p.pm_bq + (c0 % p.pm_bq);
            const int4* m4 = reinterpret_cast<const int4*>(mrow);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const int4 mv = __ldg(m4 + t);
              const uint32_t wd[4] = {(uint32_t)mv.x, (uint32_t)mv.y, (uint32_t)mv.z, (uint32_t)mv.w};
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (((wd[j >> 2] >> ((j & 3) * 8)) & 0xffu) == 0u) pr[t * 16 + j] = kMaskedLogit;
            }
          }
        }
        if (has_seg && !((ent.y >> 4) & 1)) {  // (bit set: the whole tile lies inside one segment)
          const int4* sg4 = reinterpret_cast<const int4*>(other_seg + c0);
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const int4 sv = __ldg(sg4 + t);
            if (sv.x != own_seg) pr[t * 4 + 0] = kMaskedLogit;
            if (sv.y != own_seg) pr[t * 4 + 1] = kMaskedLogit;
            if (sv.z != own_seg) pr[t * 4 + 2] = kMaskedLogit;
            if (sv.w != own_seg) pr[t * 4 + 3] = kMaskedLogit;
          }
        }
        // P = exp2(c * s - lse * log2 e); with a soft cap dS carries the factor 1 - tanh^2 (masked
        // entries hold -1e30 in place of tanh; the clamp keeps their factor finite, their p is 0)
        float fac[kSoftCap ? 64 : 1];
        const float4* nl4 = reinterpret_cast<const float4*>(p.nlse2 + stat_base + c0);  // dk / dv: per column
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          float4 nl = make_float4(row_nlse2, row_nlse2, row_nlse2, row_nlse2);
          if (kPass != kWideDq) nl = __ldg(nl4 + t);
          if constexpr (kSoftCap) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float th = fmaxf(pr[4 * t + u], -1.0f);
              fac[4 * t + u] = fmaf(-th, th, 1.0f);
            }
          }
          pr[4 * t + 0] = ex2(fmaf(pr[4 * t + 0], c, nl.x));
          pr[4 * t + 1] = ex2(fmaf(pr[4 * t + 1], c, nl.y));
          pr[4 * t + 2] = ex2(fmaf(pr[4 * t + 2], c, nl.z));
          pr[4 * t + 3] = ex2(fmaf(pr[4 * t + 3], c, nl.w));
        }
        uint32_t pk[32];
        if (kPass == kWideDv) {
#pragma unroll
          for (int j = 0; j < 32; ++j) pk[j] = pack_bf16(pr[2 * j], pr[2 * j + 1]);
        } else {
          ok = mbar_wait(&bars->dp_full, n & 1u, ab, 0xE10u);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          uint32_t v0[32], v1[32];
          tmem_ld32(t_dp + lane_addr + w * 64, v0);
          tmem_ld32(t_dp + lane_addr + w * 64 + 32, v1);
          tmem_ld_wait();
          const float4* dl4 = reinterpret_cast<const float4*>(p.delta + stat_base + c0);  // -di per column
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            float4 nd = make_float4(row_ndelta, row_ndelta, row_ndelta, row_ndelta);
            if (kPass != kWideDq) nd = __ldg(dl4 + t);
            const uint32_t* v = t < 8 ? v0 : v1;
            const int b = (t & 7) * 4;
            float d0 = pr[4 * t + 0] * (__uint_as_float(v[b + 0]) + nd.x);
            float d1 = pr[4 * t + 1] * (__uint_as_float(v[b + 1]) + nd.y);
            float d2 = pr[4 * t + 2] * (__uint_as_float(v[b + 2]) + nd.z);
            float d3 = pr[4 * t + 3] * (__uint_as_float(v[b + 3]) + nd.w);
            if constexpr (kSoftCap) {
              d0 *= fac[4 * t + 0];
              d1 *= fac[4 * t + 1];
              d2 *= fac[4 * t + 2];
              d3 *= fac[4 * t + 3];
            }
            pk[2 * t] = pack_bf16(d0, d1);
            pk[2 * t + 1] = pack_bf16(d2, d3);
          }
        }
        tmem_st32(t_sn + lane_addr + packed_col(w), pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->ds_full[sb]);
      }
    }

    // epilogue: warpgroup w stores the output's panel w (columns 128 w .. 128 w + 127)
    const int out_cols = kPass == kWideDv ? p.d_v : p.d_qk;
    const float mul = kPass == kWideDv ? 1.0f : p.scale;
    __nv_bfloat16* dst = p.out0 + (int64_t)batch * p.out0_sb + (int64_t)own_head * p.out0_sh + (int64_t)row * p.out0_ss;
    if (n_steps > 0) {
      if (ok) {
        ok = mbar_wait(&bars->acc_done, 0, ab, 0xE20u);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        for (int g = 0; g < 4; ++g) {
          const int col = w * kHeadDim + g * 32;
          if (col >= out_cols) break;
          uint32_t v[32];
          tmem_ld32(t_out + lane_addr + col, v);
          tmem_ld_wait();
          store_row_half(dst + col, v, mul, col, out_cols);
        }
      }
    } else {
      uint32_t v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0u;
      for (int g = 0; g < 4; ++g) {
        const int col = w * kHeadDim + g * 32;
        if (col >= out_cols) break;
        store_row_half(dst + col, v, 0.f, col, out_cols);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

template <int kPass>
static int launch_wide_pass(const CUtensorMap& tm_q, const CUtensorMap& tm_do, const CUtensorMap& tm_k,
                            const CUtensorMap& tm_v, const BwdParams& p, bool soft_cap, cudaStream_t stream) {
  if ((int64_t)p.n_rows * p.n_groups > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;
  const void* fn = soft_cap ? (const void*)splash_bwd_wide_kernel<kPass, true> : (const void*)splash_bwd_wide_kernel<kPass, false>;
  {
    static std::mutex attr_mu;
    static bool attr_done[64][2] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SPLASH_ERR_CUDA;
    std::lock_guard<std::mutex> lock(attr_mu);
    if (!attr_done[dev][soft_cap ? 1 : 0]) {
      if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kWideBwdSmemBytes) != cudaSuccess)
        return SPLASH_ERR_CUDA;
      attr_done[dev][soft_cap ? 1 : 0] = true;
    }
  }
  const dim3 grid((unsigned)(p.n_rows * p.n_groups), 1u, 1u);
  if (soft_cap)
    splash_bwd_wide_kernel<kPass, true><<<grid, kBwdThreads, kWideBwdSmemBytes, stream>>>(tm_q, tm_do, tm_k, tm_v, p);
  else
    splash_bwd_wide_kernel<kPass, false><<<grid, kBwdThreads, kWideBwdSmemBytes, stream>>>(tm_q, tm_do, tm_k, tm_v, p);
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}

int launch_bwd_wide(const CUtensorMap& tm_q, const CUtensorMap& tm_do, const CUtensorMap& tm_k,
                    const CUtensorMap& tm_v, BwdParams p, const SplashBwdArgs& a, bool soft_cap,
                    uint32_t launch_mask, cudaStream_t stream) {
  const int64_t B = a.q.size[0], Hq = a.q.size[1], Sq = a.q.size[2], Hkv = a.k.size[1], Skv = a.k.size[2];
  const int64_t row_bytes = 2 * (a.q.size[3] + a.v.size[3]);  // one token of k + v, or of q + do
  int st;
  auto use_schedule = [&](const SplashDeviceSchedule& s) {
    p.row_ptr = s.row_ptr;
    p.entries = reinterpret_cast<const int4*>(s.entries);
    p.row_order = s.row_order;
    p.row_end = s.row_end;
    p.entries_per_batch = s.entries_per_batch;
    p.pmb = s.partial_mask_blocks;
    p.pm_bq = s.block_q > 0 ? s.block_q : kTile;
    p.pm_bkv = s.block_kv > 0 ? s.block_kv : kTile;
    p.n_rows = s.n_rows;
  };
  auto use_output = [&](const SplashTensor& t) {
    p.out0 = static_cast<__nv_bfloat16*>(t.data);
    p.out0_sb = t.stride[0];
    p.out0_sh = t.stride[1];
    p.out0_ss = t.stride[2];
    p.out1 = nullptr;
    p.out1_sb = p.out1_sh = p.out1_ss = 0;
  };
  p.dq_acc = nullptr;
  if (launch_mask & 2u) {
    use_schedule(a.sched_dq);
    use_output(a.dq);
    p.n_groups = (int)(Hq * B);  // the q heads of one kv head stream the same K / V
    p.chunk_groups = chunk_groups_for(Skv * row_bytes / (Hq / Hkv), p.n_groups, Hq / Hkv);
    if ((st = launch_wide_pass<kWideDq>(tm_q, tm_do, tm_k, tm_v, p, soft_cap, stream))) return st;
  }
  if (launch_mask & 4u) {
    use_schedule(a.sched_dkv);
    p.n_groups = (int)(Hkv * B);  // the kv tiles of one (batch, kv head) stream the same Q / dO of its q heads
    p.chunk_groups = chunk_groups_for((Hq / Hkv) * Sq * row_bytes, p.n_groups, 1);
    use_output(a.dk);
    if ((st = launch_wide_pass<kWideDk>(tm_q, tm_do, tm_k, tm_v, p, soft_cap, stream))) return st;
    use_output(a.dv);
    if ((st = launch_wide_pass<kWideDv>(tm_q, tm_do, tm_k, tm_v, p, soft_cap, stream))) return st;
  }
  return SPLASH_OK;
}

}  // namespace sb
