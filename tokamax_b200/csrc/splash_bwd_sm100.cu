// Splash attention backward for sm_100a: bf16 inputs, head_dim 128, fp32 accumulation.
//
// Two forms.  The split form is atomic-free and bitwise repeatable in all three gradients:
//   1. delta      : -di[b,h,q] = -sum_d o * do  (stored negated: dP + (-di) is an add, which has a
//                   two-wide form)                                   (HBM-bound elementwise pass)
//   2. dq kernel  : one CTA per (q tile, q head).  Per kv tile: S = Q K^T, dP = dO V^T,
//                   dS = P o (dP - di), dQ += dS K.
//   3. dkv kernel : one CTA per (kv tile, kv head).  Loops over the q heads that share the kv
//                   head and their active q tiles: S^T = K Q^T, dP^T = V dO^T, dV += P^T dO,
//                   dK += dS^T Q.  The whole GQA group is summed in the CTA's fp32 TMEM
//                   accumulators, so dK/dV need no atomics and no second pass.
// The fused form (SPLASH_BWD_FUSED_DQ) is what the reference's live backward does — one kernel,
// five matmuls per live block (splash_attention_kernel.py:1234-1459, dq partials :1395-1410
// reduced at :1864): the dkv kernel also forms dQ_partial = dS K for every (q tile, kv tile) pair
// it visits, from the dS^T tile it already holds in shared memory, and adds it into an fp32 dQ
// image in global memory (vector red.add from four drain warps); a last HBM-bound pass scales
// and casts that image to bf16.  S and dP are then computed once per pair instead of twice (5
// tile-MMAs instead of 7).  dK / dV stay atomic-free and repeatable; dQ's fp32 sums arrive in an
// order that varies from run to run, so its last bits are not repeatable in this form.
// P (and dS in the dq kernel) is written back to TMEM as bf16 and consumed as the A operand of the
// next MMA; the dkv kernel's dS^T goes through shared memory instead, which frees its TMEM columns
// a step earlier.  K, V, Q and dO tiles are each staged once by TMA and read both K-major and
// MN-major from the same 128-byte-swizzled shared-memory image.
//
// Arithmetic follows the reference backward
// (tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_kernel.py:1234-1459 and
// base.py:115-173): P = exp(S - logsumexp), dS = (dP - di) * P, with the softmax scale applied
// in fp32 inside the kernels.
#include <mutex>

#include "splash_common.cuh"
#include "splash_bwd_params.cuh"

namespace sb {

constexpr int kBwdStages = 4;
constexpr int kDqStages = 5;  // K/V ring of the dq kernel: 2.5 steps of look-ahead

// ------------------------------------------------------------------------------------------
// delta = rowsum(o * do)
// ------------------------------------------------------------------------------------------
struct DeltaParams {
  const __nv_bfloat16* o;
  const __nv_bfloat16* d_o;
  int64_t o_sb, o_sh, o_ss, do_sb, do_sh, do_ss;
  float* delta;      // [B, Hq, Sq]  -sum_d(o * do)
  const float* lse;  // [B, Hq, Sq] natural log
  float* nlse2;      // [B, Hq, Sq]  -lse * log2(e): the exponent offset the MMA kernels subtract
  int q_heads, q_len;
  int d_v;  // columns of o / do
  int64_t n_rows;
  // fused backward: the fp32 dQ image (one 128 x 128 tile per 128 rows, [col / 4][row][col % 4])
  // that the reds of the dkv kernel add into; this pass clears it on the way.  nullptr: none.
  float* dq_image;
};

// 64 rows per block: a warp takes eight rows, half a warp per row (16 lanes x 16 bytes = one row of
// 128 bf16), four rows deep, with all eight 16-byte loads of a lane in flight before the first is
// used (the pass is a pure stream: 512 bytes read and 8 written per row).
constexpr int kDeltaRowsPerBlock = 64;
__global__ void __launch_bounds__(256) splash_delta_kernel(const DeltaParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane & 15, half = lane >> 4;
  const int64_t row0 = (int64_t)blockIdx.x * kDeltaRowsPerBlock + warp * 8 + half;
  if (p.dq_image != nullptr) {
    // The block's 64 rows are half of one image tile (q_len is a multiple of 128): for each of the
    // 32 four-column groups a run of 64 rows x 16 bytes.  256 threads x 8 stores of 16 bytes.
    const int64_t first = (int64_t)blockIdx.x * kDeltaRowsPerBlock;
    float* tile = p.dq_image + (first / kTile) * (int64_t)(kTile * kHeadDim) + (first % kTile) * 4;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = i * 256 + threadIdx.x;  // 0 .. 2047: (column group, row) of the half tile
      const int cg = idx >> 6, r = idx & 63;
      *reinterpret_cast<uint4*>(tile + (int64_t)cg * (kTile * 4) + r * 4) = zero;
    }
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  // one pass per 128 columns (a second one only for head dims above 128)
  for (int c0 = 0; c0 < p.d_v; c0 += kHeadDim) {
    uint4 a[4], g[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t row = row0 + 2 * i;
      a[i] = make_uint4(0u, 0u, 0u, 0u);
      g[i] = a[i];
      if (row < p.n_rows && c0 + sub * 8 < p.d_v) {
        const int q = (int)(row % p.q_len);
        const int64_t bh = row / p.q_len;
        const int h = (int)(bh % p.q_heads);
        const int64_t b = bh / p.q_heads;
        a[i] = __ldg(reinterpret_cast<const uint4*>(p.o + b * p.o_sb + h * p.o_sh + (int64_t)q * p.o_ss + c0) + sub);
        g[i] = __ldg(reinterpret_cast<const uint4*>(p.d_o + b * p.do_sb + h * p.do_sh + (int64_t)q * p.do_ss + c0) + sub);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t aw[4] = {a[i].x, a[i].y, a[i].z, a[i].w}, gw[4] = {g[i].x, g[i].y, g[i].z, g[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&aw[j]);
        const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(&gw[j]);
        acc[i] = fmaf(__bfloat162float(x.x), __bfloat162float(y.x), acc[i]);
        acc[i] = fmaf(__bfloat162float(x.y), __bfloat162float(y.y), acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float sum = acc[i];
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const int64_t row = row0 + 2 * i;
    if (sub == 0 && row < p.n_rows) {
      p.delta[row] = -sum;
      // Rows that never met a live key carry the mask value as logsumexp; -inf keeps their
      // probabilities at exactly zero instead of overflowing the product to +inf.
      const float lse = p.lse[row];
      p.nlse2[row] = lse < -1.0e20f ? -INFINITY : -lse * kLog2e;
    }
  }
}

// ------------------------------------------------------------------------------------------
// shared pieces of the two MMA kernels
// ------------------------------------------------------------------------------------------
struct BwdBarriers {
  uint64_t stat_full[2];              // stationary operand tiles
  uint64_t ring_full[kDqStages];
  uint64_t ring_empty[kDqStages];
  uint64_t s_full[2];
  uint64_t dp_full;
  uint64_t p_full;                    // dkv: P^T ready; dq: unused
  uint64_t ds_full;
  uint64_t acc_done;
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t early_exit;
};

constexpr int kDqSmemBytes = (2 + kDqStages) * kTileBytes + 1024 + 1024;

// ------------------------------------------------------------------------------------------
// dq kernel
// ------------------------------------------------------------------------------------------
// TMEM: S0 [0,128) | S1 [128,256) | dP [256,384) | dQ [384,512)
template <bool kSoftCap>
__global__ void __launch_bounds__(kBwdThreads, 1)
splash_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;
  uint8_t* do_smem = smem + kTileBytes;
  uint8_t* ring = smem + 2 * kTileBytes;
  BwdBarriers* bars = reinterpret_cast<BwdBarriers*>(smem + (2 + kDqStages) * kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const CtaWork work = cta_work(p.row_order, p.n_rows, p.n_groups, p.chunk_groups, true);
  const int q_tile = work.row;
  const int head = work.group % p.q_heads;
  const int batch = work.group / p.q_heads;
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int ebeg = p.row_ptr[q_tile];
  const int eend = p.row_end ? p.row_end[(int64_t)batch * p.n_rows + q_tile] : p.row_ptr[q_tile + 1];
  const int4* entries = p.entries + (int64_t)batch * p.entries_per_batch;
  const int n_ent = eend - ebeg;

  if (threadIdx.x == 0) {
    bars->early_exit = *reinterpret_cast<volatile uint32_t*>(p.err);
    bars->abort_flag = 0;
    mbar_init(&bars->stat_full[0], 1);
    mbar_init(&bars->stat_full[1], 1);
    for (int s = 0; s < kDqStages; ++s) {
      mbar_init(&bars->ring_full[s], 1);
      mbar_init(&bars->ring_empty[s], 1);
    }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_full, 8);
    mbar_init(&bars->ds_full, 8);  // one arrival per compute warp
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

  if (warp >= 8) {
   setmaxnreg_dec<kIssueRegs>();
   if (warp == 8) {
    if (lane == 0 && n_ent > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      // tiles are two 64-column halves; with at most 64 real columns the second is never read
      const bool qk2 = p.d_qk > 64, v2 = p.d_v > 64;
      mbar_arrive_expect_tx(&bars->stat_full[0], qk2 ? kTileBytes : kHalfBytes);
      tma_load_4d(q_smem, &tm_q, &bars->stat_full[0], 0, q_tile * kTile, head, batch);
      if (qk2) tma_load_4d(q_smem + kHalfBytes, &tm_q, &bars->stat_full[0], 64, q_tile * kTile, head, batch);
      mbar_arrive_expect_tx(&bars->stat_full[1], v2 ? kTileBytes : kHalfBytes);
      tma_load_4d(do_smem, &tm_do, &bars->stat_full[1], 0, q_tile * kTile, head, batch);
      if (v2) tma_load_4d(do_smem + kHalfBytes, &tm_do, &bars->stat_full[1], 64, q_tile * kTile, head, batch);
      uint32_t it = 0;
      bool ok = true;
      for (int e = ebeg; e < eend && ok; ++e) {
        const int col = entries[e].x;
        for (int kv = 0; kv < 2 && ok; ++kv, ++it) {
          const uint32_t s = it % kDqStages;
          ok = mbar_wait(&bars->ring_empty[s], ((it / kDqStages) & 1u) ^ 1u, ab, 0x1100u + s);
          if (!ok) break;
          uint8_t* dst = ring + s * kTileBytes;
          const CUtensorMap* tm = kv == 0 ? &tm_k : &tm_v;
          const bool two = kv == 0 ? qk2 : v2;
          mbar_arrive_expect_tx(&bars->ring_full[s], two ? kTileBytes : kHalfBytes);
          tma_load_4d(dst, tm, &bars->ring_full[s], 0, col * kTile, kv_head, batch);
          if (two) tma_load_4d(dst + kHalfBytes, tm, &bars->ring_full[s], 64, col * kTile, kv_head, batch);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0 && n_ent > 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(kTile, kTile, false, false);
      // N of dQ += dS K: dq's columns — 128, or 64 when q / k have at most 64
      const uint32_t idesc_mn = make_idesc_bf16(kTile, p.d_qk <= 64 ? 64 : kHeadDim, false, true);
      const uint32_t q_addr = smem_u32(q_smem), do_addr = smem_u32(do_smem), ring_addr = smem_u32(ring);
      const uint32_t t_dp = tmem + 2 * kTile, t_dq = tmem + 3 * kTile;
      auto ss_kmajor = [&](uint32_t d, uint32_t a0, uint32_t b0, int nk) {
        const SmemDesc da = make_smem_desc_sw128(a0, 16, 1024), db = make_smem_desc_sw128(b0, 16, 1024);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (nk != 8 && k >= nk) break;  // head dims below 128: the remaining slices multiply zeros
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          umma_ss(d, desc_at(da, off), desc_at(db, off), idesc_kk, k > 0 ? 1u : 0u);
        }
      };
      auto ring_wait = [&](uint32_t it, uint32_t tag) {
        return mbar_wait(&bars->ring_full[it % kDqStages], (it / kDqStages) & 1u, ab, tag);
      };
      bool ok = mbar_wait(&bars->stat_full[0], 0, ab, 0x1200u) && mbar_wait(&bars->stat_full[1], 0, ab, 0x1201u);
      // prologue: S_0, dP_0
      ok = ok && ring_wait(0, 0x1210u);
      if (ok) {
        mma_issue_fence();
        ss_kmajor(tmem, q_addr, ring_addr, p.nk_qk);
        tc_commit(&bars->s_full[0]);
      }
      ok = ok && ring_wait(1, 0x1211u);
      if (ok) {
        mma_issue_fence();
        ss_kmajor(t_dp, do_addr, ring_addr + kTileBytes, p.nk_v);
        tc_commit(&bars->dp_full);
        tc_commit(&bars->ring_empty[1]);
      }
      for (int n = 0; n < n_ent && ok; ++n) {
        const bool has_next = n + 1 < n_ent;
        const uint32_t it_k = 2 * n, it_kn = 2 * n + 2, it_vn = 2 * n + 3;
        if (has_next) {
          ok = ring_wait(it_kn, 0x1220u);
          if (!ok) break;
          mma_issue_fence();
          ss_kmajor(tmem + ((n + 1) & 1) * kTile, q_addr, ring_addr + (it_kn % kDqStages) * kTileBytes, p.nk_qk);
          tc_commit(&bars->s_full[(n + 1) & 1]);
        }
        ok = mbar_wait(&bars->ds_full, n & 1u, ab, 0x1230u);
        if (!ok) break;
        mma_issue_fence();
        {
          // dQ += dS_n K_n : A = packed dS in the S buffer, B = K tile read MN-major.
          const uint32_t a_base = tmem + (n & 1) * kTile;
          const SmemDesc db = make_smem_desc_sw128(ring_addr + (it_k % kDqStages) * kTileBytes, kHalfBytes, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_ts(t_dq, a_base + packed_a_col(k), desc_at(db, k * 2048), idesc_mn, (n > 0 || k > 0) ? 1u : 0u);
          tc_commit(&bars->ring_empty[it_k % kDqStages]);
        }
        if (has_next) {
          ok = ring_wait(it_vn, 0x1240u);
          if (!ok) break;
          mma_issue_fence();
          ss_kmajor(t_dp, do_addr, ring_addr + (it_vn % kDqStages) * kTileBytes, p.nk_v);
          tc_commit(&bars->dp_full);
          tc_commit(&bars->ring_empty[it_vn % kDqStages]);
        }
      }
      tc_commit(&bars->acc_done);
    }
   }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    setmaxnreg_inc<kComputeRegs>();
    const int w = warp >> 2;       // column half this warpgroup owns
    const int wq = warp & 3;
    const int r = wq * 32 + lane;  // q row within the tile
    const int q_row = q_tile * kTile + r;
    const int qi = p.q_sequence ? p.q_sequence[q_row] : q_row;
    const RowInterval iv = mask_fn_interval(p.fn, qi);
    const bool has_seg = p.q_seg != nullptr;
    const int q_seg = has_seg ? p.q_seg[(int64_t)batch * p.q_len + q_row] : 0;
    const int32_t* kv_seg_row = has_seg ? p.kv_seg + (int64_t)batch * p.kv_len : nullptr;
    const int64_t stat = ((int64_t)batch * p.q_heads + head) * p.q_len + q_row;
    const float nlse2 = p.nlse2[stat];
    const float ndelta = p.delta[stat];  // -di
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c = kSoftCap ? p.soft_cap * kLog2e : p.scale_log2;
    bool ok = true;

    int4 ent_next = n_ent > 0 ? entries[ebeg] : make_int4(0, 0, 0, 0);
    for (int n = 0; n < n_ent; ++n) {
      const int4 ent = ent_next;
      if (n + 1 < n_ent) ent_next = entries[ebeg + n + 1];  // fetched a step ahead of its use
      const int st = ent.y & 3;
      const int kv0 = ent.x * kTile + w * 64;
      const uint32_t t_s = tmem + lane_addr + (n & 1) * kTile;
      ok = mbar_wait(&bars->s_full[n & 1], (n >> 1) & 1u, ab, 0x1400u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float pr[64];
      {
        uint32_t v0[32], v1[32];
        tmem_ld32(t_s + w * 64, v0);
        tmem_ld32(t_s + w * 64 + 32, v1);
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
          const int lo_rel = iv.lo <= kv0 ? 0 : iv.lo - kv0;
          const int hi_rel = iv.hi >= kv0 + 63 ? 63 : iv.hi - kv0;
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (j < lo_rel || j > hi_rel) pr[j] = kMaskedLogit;
        } else {
          const int8_t* mrow = p.pmb + ((int64_t)ent.z * p.pm_bq + (q_row % p.pm_bq)) * p.pm_bkv +
                               (kv0 % p.pm_bkv);
          const int4* m4 = reinterpret_cast<const int4*>(mrow);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int4 mv = __ldg(m4 + g);
            const uint32_t wd[4] = {(uint32_t)mv.x, (uint32_t)mv.y, (uint32_t)mv.z, (uint32_t)mv.w};
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (((wd[j >> 2] >> ((j & 3) * 8)) & 0xffu) == 0u) pr[g * 16 + j] = kMaskedLogit;
          }
        }
      }
      if (has_seg && !((ent.y >> 4) & 1)) {  // (bit set: the whole tile lies inside one segment)
        const int4* sg4 = reinterpret_cast<const int4*>(kv_seg_row + kv0);
#pragma unroll
        for (int g = 0; g < 16; ++g) {
          const int4 sv = __ldg(sg4 + g);
          if (sv.x != q_seg) pr[g * 4 + 0] = kMaskedLogit;
          if (sv.y != q_seg) pr[g * 4 + 1] = kMaskedLogit;
          if (sv.z != q_seg) pr[g * 4 + 2] = kMaskedLogit;
          if (sv.w != q_seg) pr[g * 4 + 3] = kMaskedLogit;
        }
      }
      if constexpr (kSoftCap) {
        // p * (1 - tanh^2): the chain factor of the cap rides on p (masked entries hold -1e30
        // in place of tanh; the clamp keeps their factor finite, their p is 0)
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float t = fmaxf(pr[j], -1.0f);
          pr[j] = ex2(fmaf(pr[j], c, nlse2)) * fmaf(-t, t, 1.0f);
        }
      } else {
        // issue-bound: two-wide fp32 fma for the exponent arguments
        const float2 c2 = make_float2(c, c), nl2 = make_float2(nlse2, nlse2);
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          const float2 x = __ffma2_rn(make_float2(pr[j], pr[j + 1]), c2, nl2);
          pr[j] = ex2(x.x);
          pr[j + 1] = ex2(x.y);
        }
      }

      ok = mbar_wait(&bars->dp_full, n & 1u, ab, 0x1410u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t pk[32];
      {
        uint32_t v0[32], v1[32];
        tmem_ld32(tmem + lane_addr + 2 * kTile + w * 64, v0);
        tmem_ld32(tmem + lane_addr + 2 * kTile + w * 64 + 32, v1);
        tmem_ld_wait();
        const float2 nd2 = make_float2(ndelta, ndelta);
#pragma unroll
        for (int j = 0; j < 16; ++j) {  // dS = p * (dP - di), two elements per instruction
          const float2 a = __fmul2_rn(make_float2(pr[2 * j], pr[2 * j + 1]),
                                      __fadd2_rn(make_float2(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1])), nd2));
          const float2 b = __fmul2_rn(make_float2(pr[32 + 2 * j], pr[32 + 2 * j + 1]),
                                      __fadd2_rn(make_float2(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1])), nd2));
          pk[j] = pack_bf16(a.x, a.y);
          pk[16 + j] = pack_bf16(b.x, b.y);
        }
      }
      tmem_st32(t_s + packed_col(w), pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_full);
    }

    // epilogue
    __nv_bfloat16* dst = p.out0 + (int64_t)batch * p.out0_sb + (int64_t)head * p.out0_sh +
                         (int64_t)q_row * p.out0_ss + w * 64;
    if (n_ent > 0) {
      if (ok) {
        ok = mbar_wait(&bars->acc_done, 0, ab, 0x1500u);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t v[32];
          tmem_ld32(tmem + lane_addr + 3 * kTile + w * 64 + g * 32, v);
          tmem_ld_wait();
          store_row_half(dst + g * 32, v, p.scale, w * 64 + g * 32, p.d_qk);
        }
      }
    } else {
      uint32_t v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0u;
      store_row_half(dst, v, 0.f, w * 64, p.d_qk);
      store_row_half(dst + 32, v, 0.f, w * 64 + 32, p.d_qk);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// dkv kernel
// ------------------------------------------------------------------------------------------
// 16 compute warps (thread = kv row x one 32-column quarter of the q tile) keep the P^T / dS^T
// phases short; warp 16 feeds TMA, warp 17 issues MMAs, warps 18-19 are idle (they complete the
// fifth warpgroup).
constexpr int kDkvThreads = 640;
constexpr int kDkvTmaWarp = 16;
constexpr int kDkvMmaWarp = 17;
// Fused form: warps 20-23 drain the per-pair dQ tile from TMEM into the fp32 image.  768 threads
// start at 80 registers.  Registers live in four banks, one per scheduler, and warp w draws on bank
// w mod 4, so every bank serves four compute warps, one warp of the issuing warpgroup and one
// drain warp: 6 x 80 at launch, 4 x 88 + 80 + 48 after the hand-over (the sum per bank has to stay
// at what the launch gave it, or the increase never completes).
constexpr int kFusedThreads = 768;
constexpr int kDkvDrainWarp = 20;
constexpr int kFusedComputeRegs = 88;
constexpr int kFusedDrainRegs = 48;
constexpr int kDqTileFloats = kTile * kHeadDim;
// No register hand-over here: at 640 threads every thread gets 96 registers, which the compute
// warps fit in, and the MMA / TMA threads keep their loop state in registers instead of spilling
// it (with 56 registers the issue loop reloaded descriptor bases from local memory).

// One CTA = one kv tile of one (batch, kv head); the q heads of the GQA group and the active q
// tiles are looped inside and dK / dV of the whole group accumulate in TMEM in fp32 (no atomics,
// bitwise repeatable).  A q tile is processed whole: the score MMAs run with N = 128 (an N = 64 SS
// MMA reads 6 KB of shared memory for 32 cycles of tensor time and so runs at about 60 % of the
// N = 128 rate; a version that double-buffered 64-column halves of the q tile was 21 % slower).
//   TMEM: S^T [0,128) | dP^T [128,256) | dK [256,384) | dV [384,512)
// S^T and dP^T are single-buffered.  P^T goes back to TMEM over S^T (A operand of dV += P^T dO);
// dS^T goes to shared memory in the K-major 128-byte-swizzled layout of an operand tile (A operand
// of dK += dS^T Q), which frees the dP^T columns for the next step as soon as they have been
// read.  Issue order of step n:  wait P^T(n) | dV(n) | S^T(n+1) | wait dS^T(n) | dK(n) | dP^T(n+1)
// — the tensor pipe executes in order, so S^T(n+1) cannot overtake dV(n)'s read of P^T(n), and
// dP^T(n+1) is issued only after the compute warps have consumed dP^T(n).
constexpr int kDkvStatsBytes = (kBwdStages / 2) * 2 * kTile * 4;
constexpr int kDkvSmemBytes = (3 + kBwdStages) * kTileBytes + kDkvStatsBytes + 512;

struct DkvBarriers {
  uint64_t stat_full[2];
  uint64_t ring_full[kBwdStages];
  uint64_t ring_empty[kBwdStages];
  uint64_t st_full;
  uint64_t dpt_full;
  uint64_t p_full;
  uint64_t ds_full;
  uint64_t ds_free;   // dK(n) has finished reading the dS^T tile in shared memory
  uint64_t acc_done;
  uint64_t dq_full;   // fused: dQ_partial(n) is complete in the dP^T columns
  uint64_t dq_free;   // fused: the drain warps have read it out (4 arrivals)
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t early_exit;
};
static_assert(sizeof(DkvBarriers) <= 512, "barrier block");

template <bool kSoftCap, bool kFuseDq>
__global__ void __launch_bounds__(kFuseDq ? kFusedThreads : kDkvThreads, 1)
splash_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* k_smem = smem;
  uint8_t* v_smem = smem + kTileBytes;
  uint8_t* ds_smem = smem + 2 * kTileBytes;
  uint8_t* ring = smem + 3 * kTileBytes;
  float* stats = reinterpret_cast<float*>(smem + (3 + kBwdStages) * kTileBytes);
  DkvBarriers* bars = reinterpret_cast<DkvBarriers*>(smem + (3 + kBwdStages) * kTileBytes + kDkvStatsBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const CtaWork work = cta_work(p.row_order, p.n_rows, p.n_groups, p.chunk_groups, false);
  const int kv_tile = work.row;
  const int kv_head = work.group % p.kv_heads;
  const int batch = work.group / p.kv_heads;
  const int group = p.q_heads / p.kv_heads;
  const int ebeg = p.row_ptr[kv_tile];
  const int eend = p.row_end ? p.row_end[(int64_t)batch * p.n_rows + kv_tile] : p.row_ptr[kv_tile + 1];
  const int4* entries = p.entries + (int64_t)batch * p.entries_per_batch;
  const int n_ent = eend - ebeg;
  const int n_steps = n_ent * group;

  if (threadIdx.x == 0) {
    // The operand tiles need a 1024-byte aligned base for the 128-byte swizzle; there is no
    // slack in the allocation to fix it up, so a misaligned window is reported, not used.
    uint32_t bad = *reinterpret_cast<volatile uint32_t*>(p.err);
    if ((smem_u32(smem) & 1023u) != 0u) {
      if (atomicCAS(p.err, 0u, 2u) == 0u) {
        p.err[1] = blockIdx.x;
        p.err[2] = 0x2f00u;
        p.err[3] = smem_u32(smem);
      }
      bad = 2u;
    }
    bars->early_exit = bad;
    bars->abort_flag = 0;
    mbar_init(&bars->stat_full[0], 1);
    mbar_init(&bars->stat_full[1], 1);
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(&bars->ring_full[s], 1);
      mbar_init(&bars->ring_empty[s], 1);
    }
    mbar_init(&bars->st_full, 1);
    mbar_init(&bars->dpt_full, 1);
    mbar_init(&bars->p_full, 16);   // one arrival per compute warp
    mbar_init(&bars->ds_full, 16);
    mbar_init(&bars->ds_free, 1);
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_free, 4);
    mbar_fence_init();
  }
  __syncthreads();
  if (bars->early_exit != 0) return;
  if (warp == kDkvMmaWarp) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  AbortCtx ab{&bars->abort_flag, p.err};

  if (kFuseDq && warp >= kDkvDrainWarp) {
    // ------------------------------------------------------------------ dQ drain (fused form)
    // Thread = q row of the pair's dQ tile (TMEM lane) x all 128 head-dim columns, read 32 at a
    // time and added to the fp32 image with four-wide reds.  The TMEM columns are handed back
    // to the issuing thread as soon as the last load has completed, before the last reds go out.
    setmaxnreg_dec<kFusedDrainRegs>();
    const int wq = warp & 3;
    const int r = wq * 32 + lane;
    const uint32_t t_dq = tmem + ((uint32_t)(wq * 32) << 16) + kTile;
    const int n_q_tiles = p.q_len / kTile;
    bool ok = true;
    uint32_t n = 0;
    for (int g = 0; g < group && ok; ++g) {
      const int head = kv_head * group + g;
      float* head_base = p.dq_acc + ((int64_t)batch * p.q_heads + head) * n_q_tiles * (int64_t)kDqTileFloats + r * 4;
      for (int e = ebeg; e < eend && ok; ++e, ++n) {
        float* dst = head_base + (int64_t)entries[e].x * kDqTileFloats;
        ok = mbar_wait(&bars->dq_full, n & 1u, ab, 0x3600u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const int last = p.d_qk <= 64 ? 1 : 3;  // 32-column chunks beyond dq's columns hold nothing
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (c > last) break;
          uint32_t v[32];
          tmem_ld32(t_dq + c * 32, v);
          tmem_ld_wait();
          if (c == last) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->dq_free);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            red_add_v4(dst + (c * 8 + j) * (kTile * 4), __uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                       __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
        }
      }
    }
  } else if (warp >= 16) {
   if (warp == kDkvTmaWarp) {
    if (lane == 0 && n_steps > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      // tiles are two 64-column halves; with at most 64 real columns the second is never read
      const bool qk2 = p.d_qk > 64, v2 = p.d_v > 64;
      mbar_arrive_expect_tx(&bars->stat_full[0], qk2 ? kTileBytes : kHalfBytes);
      tma_load_4d(k_smem, &tm_k, &bars->stat_full[0], 0, kv_tile * kTile, kv_head, batch);
      if (qk2) tma_load_4d(k_smem + kHalfBytes, &tm_k, &bars->stat_full[0], 64, kv_tile * kTile, kv_head, batch);
      mbar_arrive_expect_tx(&bars->stat_full[1], v2 ? kTileBytes : kHalfBytes);
      tma_load_4d(v_smem, &tm_v, &bars->stat_full[1], 0, kv_tile * kTile, kv_head, batch);
      if (v2) tma_load_4d(v_smem + kHalfBytes, &tm_v, &bars->stat_full[1], 64, kv_tile * kTile, kv_head, batch);
      uint32_t it = 0;
      bool ok = true;
      for (int g = 0; g < group && ok; ++g) {
        const int head = kv_head * group + g;
        const int64_t stat_base = ((int64_t)batch * p.q_heads + head) * p.q_len;
        for (int e = ebeg; e < eend && ok; ++e) {
          const int qt = entries[e].x;
          for (int which = 0; which < 2 && ok; ++which, ++it) {
            const uint32_t s = it % kBwdStages;
            ok = mbar_wait(&bars->ring_empty[s], ((it / kBwdStages) & 1u) ^ 1u, ab, 0x3100u + s);
            if (!ok) break;
            uint8_t* dst = ring + s * kTileBytes;
            const CUtensorMap* tm = which == 0 ? &tm_q : &tm_do;
            const bool two = which == 0 ? qk2 : v2;
            const uint32_t tile_bytes = two ? kTileBytes : kHalfBytes;
            mbar_arrive_expect_tx(&bars->ring_full[s], which == 0 ? tile_bytes + 2 * kTile * 4 : tile_bytes);
            tma_load_4d(dst, tm, &bars->ring_full[s], 0, qt * kTile, head, batch);
            if (two) tma_load_4d(dst + kHalfBytes, tm, &bars->ring_full[s], 64, qt * kTile, head, batch);
            if (which == 0) {  // the step's statistics ride on the Q slot's barrier
              float* sdst = stats + (s / 2) * 2 * kTile;
              bulk_load(sdst, p.nlse2 + stat_base + (int64_t)qt * kTile, kTile * 4, &bars->ring_full[s]);
              bulk_load(sdst + kTile, p.delta + stat_base + (int64_t)qt * kTile, kTile * 4, &bars->ring_full[s]);
            }
          }
        }
      }
    }
  } else if (warp == kDkvMmaWarp) {
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kTile, false, false);
      // N of the accumulating MMAs = the gradient's columns: 128, or 64 when the tensor has at most 64
      const uint32_t idesc_dv = make_idesc_bf16(kTile, p.d_v <= 64 ? 64 : kHeadDim, false, true);
      const uint32_t idesc_dk = make_idesc_bf16(kTile, p.d_qk <= 64 ? 64 : kHeadDim, false, true);
      const uint32_t k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem), ds_addr = smem_u32(ds_smem);
      const uint32_t ring_addr = smem_u32(ring);
      const uint32_t t_st = tmem, t_dpt = tmem + kTile, t_dk = tmem + 2 * kTile, t_dv = tmem + 3 * kTile;
      auto slot_addr = [&](uint32_t it) { return ring_addr + (it % kBwdStages) * kTileBytes; };
      auto ring_wait = [&](uint32_t it, uint32_t tag) {
        return mbar_wait(&bars->ring_full[it % kBwdStages], (it / kBwdStages) & 1u, ab, tag);
      };
      // D = A B^T with both operands K-major (head_dim contiguous), K = head_dim
      auto issue_score = [&](uint32_t d, SmemDesc da, uint32_t b0, int nk) {
        const SmemDesc db = make_smem_desc_sw128(b0, 16, 1024);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (nk != 8 && k >= nk) break;  // head dims below 128: the remaining slices multiply zeros
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          umma_ss(d, desc_at(da, off), desc_at(db, off), idesc_s, k > 0 ? 1u : 0u);
        }
      };
      // descriptors of the stationary operands, built once
      const SmemDesc k_desc = make_smem_desc_sw128(k_addr, 16, 1024), v_desc = make_smem_desc_sw128(v_addr, 16, 1024);
      const SmemDesc ds_desc = make_smem_desc_sw128(ds_addr, 16, 1024);
      // fused form: the same two tiles seen MN-major (rows are the MMA's K dimension)
      const uint32_t idesc_dq = make_idesc_bf16(kTile, p.d_qk <= 64 ? 64 : kHeadDim, true, true);
      const SmemDesc ds_mn_desc = make_smem_desc_sw128(ds_addr, kHalfBytes, 1024);
      const SmemDesc k_mn_desc = make_smem_desc_sw128(k_addr, kHalfBytes, 1024);
      bool ok = mbar_wait(&bars->stat_full[0], 0, ab, 0x3200u) && mbar_wait(&bars->stat_full[1], 0, ab, 0x3201u);
      ok = ok && ring_wait(0, 0x3210u);
      if (ok) {
        issue_score(t_st, k_desc, slot_addr(0), p.nk_qk);
        tc_commit(&bars->st_full);
      }
      ok = ok && ring_wait(1, 0x3211u);
      if (ok) {
        issue_score(t_dpt, v_desc, slot_addr(1), p.nk_v);
        tc_commit(&bars->dpt_full);
      }
      for (int n = 0; n < n_steps && ok; ++n) {
        const uint32_t ph = (uint32_t)n & 1u;
        const uint32_t q_slot = slot_addr(2 * n), do_slot = slot_addr(2 * n + 1);
        const bool more = n + 1 < n_steps;
        ok = mbar_wait(&bars->p_full, ph, ab, 0x3220u);
        if (!ok) break;
        mma_issue_fence();
        // dV += P^T dO: A = packed bf16 P^T in TMEM (16 packed columns at the start of every
        // 32-column quarter), B = the dO tile read MN-major, K = 128 query rows in eight slices
        const SmemDesc do_mn = make_smem_desc_sw128(do_slot, kHalfBytes, 1024);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ts(t_dv, t_st + (k >> 1) * 32 + (k & 1) * 8, desc_at(do_mn, k * 2048), idesc_dv,
                  (n > 0 || k > 0) ? 1u : 0u);
        if (more) {
          ok = ring_wait(2 * (n + 1), 0x3240u);
          if (!ok) break;
          issue_score(t_st, k_desc, slot_addr(2 * (n + 1)), p.nk_qk);
          tc_commit(&bars->st_full);
        }
        ok = mbar_wait(&bars->ds_full, ph, ab, 0x3230u);
        if (!ok) break;
        mma_issue_fence();
        if constexpr (kFuseDq) {
          // dQ_partial = dS K over the dP^T columns (every compute warp has read dP^T(n) before it
          // arrived on ds_full): A = the dS^T tile read MN-major (M = q), B = the K tile read
          // MN-major (N = head dim), K = 128 kv rows in eight slices.  Issued ahead of dK so the
          // drain warps read it out while dK runs.
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_ss(t_dpt, desc_at(ds_mn_desc, k * 2048), desc_at(k_mn_desc, k * 2048), idesc_dq, k > 0 ? 1u : 0u);
          tc_commit(&bars->dq_full);
        }
        // dK += dS^T Q: A = dS^T from shared memory (K-major, two 64-column halves), B = the Q
        // tile read MN-major
        const SmemDesc q_mn = make_smem_desc_sw128(q_slot, kHalfBytes, 1024);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
          umma_ss(t_dk, desc_at(ds_desc, off), desc_at(q_mn, k * 2048), idesc_dk, (n > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&bars->ds_free);
        tc_commit(&bars->ring_empty[(2 * n) % kBwdStages]);
        tc_commit(&bars->ring_empty[(2 * n + 1) % kBwdStages]);
        if (more) {
          ok = ring_wait(2 * (n + 1) + 1, 0x3241u);
          if (!ok) break;
          if constexpr (kFuseDq) {  // the dP^T columns still hold dQ_partial(n) until it is drained
            ok = mbar_wait(&bars->dq_free, ph, ab, 0x3250u);
            if (!ok) break;
            mma_issue_fence();
          }
          issue_score(t_dpt, v_desc, slot_addr(2 * (n + 1) + 1), p.nk_v);
          tc_commit(&bars->dpt_full);
        }
      }
      tc_commit(&bars->acc_done);
    }
   }
  } else {
    // 16 warps on one 128 x 128 tile: thread = kv row (TMEM lane) x one 32-column quarter.
    if constexpr (kFuseDq) setmaxnreg_inc<kFusedComputeRegs>();
    const int cq = warp >> 2;      // column quarter 0..3
    const int wq = warp & 3;       // TMEM lane quarter
    const int r = wq * 32 + lane;  // kv row within the tile
    const int kv_row = kv_tile * kTile + r;
    const bool has_seg = p.q_seg != nullptr;
    const int kv_seg = has_seg ? p.kv_seg[(int64_t)batch * p.kv_len + kv_row] : 0;
    const int32_t* q_seg_row = has_seg ? p.q_seg + (int64_t)batch * p.q_len : nullptr;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const uint32_t t_st = tmem + lane_addr + cq * 32;
    const uint32_t t_dpt = tmem + lane_addr + kTile + cq * 32;
    // dS^T row r, columns cq*32 .. +31: 64 bytes = four 16-byte chunks of the row's 128-byte
    // segment in swizzle half cq / 2; chunk c sits at position c ^ (r mod 8)
    uint8_t* ds_row = ds_smem + (cq >> 1) * kHalfBytes + r * 128;
    const int chunk0 = (cq & 1) * 4;
    const float c = kSoftCap ? p.soft_cap * kLog2e : p.scale_log2;
    bool ok = true;
    int n = 0;

    for (int g = 0; g < group && ok; ++g) {
      int4 ent_next = n_ent > 0 ? entries[ebeg] : make_int4(0, 0, 0, 0);
      for (int e = ebeg; e < eend && ok; ++e, ++n) {
        const int4 ent = ent_next;
        if (e + 1 < eend) ent_next = entries[e + 1];
        const int st = ent.y & 3;
        const uint32_t ph = (uint32_t)n & 1u;
        const int q0 = ent.x * kTile + cq * 32;  // first q column of this thread's 32
        const uint32_t itq = 2u * (uint32_t)n;
        ok = mbar_wait(&bars->ring_full[itq % kBwdStages], (itq / kBwdStages) & 1u, ab, 0x3420u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float4* nl4 = reinterpret_cast<const float4*>(stats + ((itq % kBwdStages) / 2) * 2 * kTile + cq * 32);
        const float4* dl4 = nl4 + kTile / 4;

        ok = mbar_wait(&bars->st_full, ph, ab, 0x3400u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float pr[32];
        {
          uint32_t v[32];
          tmem_ld32(t_st, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) pr[j] = __uint_as_float(v[j]);
        }
        if constexpr (kSoftCap) {
#pragma unroll
          for (int j = 0; j < 32; ++j) pr[j] = tanh_ex2(pr[j] * p.softcap_a);
        }
        if (st == 1) {
          if (p.fn.kind != SPLASH_MASK_TABLE) {
            if (p.q_sequence == nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const RowInterval iv = mask_fn_interval(p.fn, q0 + j);
                if (kv_row < iv.lo || kv_row > iv.hi) pr[j] = kMaskedLogit;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const RowInterval iv = mask_fn_interval(p.fn, __ldg(p.q_sequence + q0 + j));
                if (kv_row < iv.lo || kv_row > iv.hi) pr[j] = kMaskedLogit;
              }
            }
          } else {
            const int8_t* mrow = p.pmb + ((int64_t)ent.z * p.pm_bkv + (kv_row % p.pm_bkv)) * p.pm_bq +
                                 (q0 % p.pm_bq);
            const int4* m4 = reinterpret_cast<const int4*>(mrow);
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int4 mv = __ldg(m4 + t);
              const uint32_t wd[4] = {(uint32_t)mv.x, (uint32_t)mv.y, (uint32_t)mv.z, (uint32_t)mv.w};
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (((wd[j >> 2] >> ((j & 3) * 8)) & 0xffu) == 0u) pr[t * 16 + j] = kMaskedLogit;
            }
          }
        }
        if (has_seg && !((ent.y >> 4) & 1)) {  // (bit set: the whole tile lies inside one segment)
          const int4* sg4 = reinterpret_cast<const int4*>(q_seg_row + q0);
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int4 sv = __ldg(sg4 + t);
            if (sv.x != kv_seg) pr[t * 4 + 0] = kMaskedLogit;
            if (sv.y != kv_seg) pr[t * 4 + 1] = kMaskedLogit;
            if (sv.z != kv_seg) pr[t * 4 + 2] = kMaskedLogit;
            if (sv.w != kv_seg) pr[t * 4 + 3] = kMaskedLogit;
          }
        }
        {
          uint32_t pk[16];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const float4 nl = nl4[t];
            float th[4];
            if constexpr (kSoftCap) {
#pragma unroll
              for (int u = 0; u < 4; ++u) th[u] = fmaxf(pr[4 * t + u], -1.0f);
            }
            const float2 xa = __ffma2_rn(make_float2(pr[4 * t + 0], pr[4 * t + 1]), make_float2(c, c),
                                         make_float2(nl.x, nl.y));
            const float2 xb = __ffma2_rn(make_float2(pr[4 * t + 2], pr[4 * t + 3]), make_float2(c, c),
                                         make_float2(nl.z, nl.w));
            pr[4 * t + 0] = ex2(xa.x);
            pr[4 * t + 1] = ex2(xa.y);
            pr[4 * t + 2] = ex2(xb.x);
            pr[4 * t + 3] = ex2(xb.y);
            pk[2 * t] = pack_bf16(pr[4 * t + 0], pr[4 * t + 1]);
            pk[2 * t + 1] = pack_bf16(pr[4 * t + 2], pr[4 * t + 3]);
            if constexpr (kSoftCap) {
#pragma unroll
              for (int u = 0; u < 4; ++u) pr[4 * t + u] *= fmaf(-th[u], th[u], 1.0f);
            }
          }
          tmem_st16(t_st, pk);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->p_full);
        }
        ok = mbar_wait(&bars->dpt_full, ph, ab, 0x3410u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t pk[16];
        {
          uint32_t v[32];
          tmem_ld32(t_dpt, v);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const float4 nd = dl4[t];  // -di of the four query columns
            const float2 a = __fmul2_rn(make_float2(pr[4 * t + 0], pr[4 * t + 1]),
                                        __fadd2_rn(make_float2(__uint_as_float(v[4 * t + 0]), __uint_as_float(v[4 * t + 1])),
                                                   make_float2(nd.x, nd.y)));
            const float2 b = __fmul2_rn(make_float2(pr[4 * t + 2], pr[4 * t + 3]),
                                        __fadd2_rn(make_float2(__uint_as_float(v[4 * t + 2]), __uint_as_float(v[4 * t + 3])),
                                                   make_float2(nd.z, nd.w)));
            pk[2 * t] = pack_bf16(a.x, a.y);
            pk[2 * t + 1] = pack_bf16(b.x, b.y);
          }
        }
        if (n > 0) {  // the previous step's dK must have finished reading the tile
          ok = mbar_wait(&bars->ds_free, (uint32_t)(n - 1) & 1u, ab, 0x3430u);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const uint4 w = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
          *reinterpret_cast<uint4*>(ds_row + (((chunk0 + ch) ^ (r & 7)) << 4)) = w;
        }
        fence_proxy_async_smem();  // generic-proxy stores -> visible to the MMA's async-proxy reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->ds_full);
      }
    }

    // epilogue: dK (scaled) and dV, 32 columns per thread
    __nv_bfloat16* dk = p.out0 + (int64_t)batch * p.out0_sb + (int64_t)kv_head * p.out0_sh +
                        (int64_t)kv_row * p.out0_ss + cq * 32;
    __nv_bfloat16* dv = p.out1 + (int64_t)batch * p.out1_sb + (int64_t)kv_head * p.out1_sh +
                        (int64_t)kv_row * p.out1_ss + cq * 32;
    if (n_steps > 0) {
      if (ok) {
        ok = mbar_wait(&bars->acc_done, 0, ab, 0x3500u);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        uint32_t v[32];
        tmem_ld32(tmem + lane_addr + 2 * kTile + cq * 32, v);
        tmem_ld_wait();
        store_row_half(dk, v, p.scale, cq * 32, p.d_qk);
        // context parallelism: the row also goes to the rank that owns it in the sequence-sharded layout
        if (p.out0_peer.ptrs) store_row_half(peer_row(p.out0_peer, batch, kv_head, kv_row) + cq * 32, v, p.scale, cq * 32, p.d_qk);
        tmem_ld32(tmem + lane_addr + 3 * kTile + cq * 32, v);
        tmem_ld_wait();
        store_row_half(dv, v, 1.0f, cq * 32, p.d_v);
        if (p.out1_peer.ptrs) store_row_half(peer_row(p.out1_peer, batch, kv_head, kv_row) + cq * 32, v, 1.0f, cq * 32, p.d_v);
      }
    } else {
      uint32_t v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0u;
      store_row_half(dk, v, 0.f, cq * 32, p.d_qk);
      store_row_half(dv, v, 0.f, cq * 32, p.d_v);
      if (p.out0_peer.ptrs) store_row_half(peer_row(p.out0_peer, batch, kv_head, kv_row) + cq * 32, v, 0.f, cq * 32, p.d_qk);
      if (p.out1_peer.ptrs) store_row_half(peer_row(p.out1_peer, batch, kv_head, kv_row) + cq * 32, v, 0.f, cq * 32, p.d_v);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kDkvMmaWarp) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------
// fused form: fp32 dQ image -> bf16 dQ
// ------------------------------------------------------------------------------------------
// One CTA per 128 x 128 tile.  A warp instruction reads eight 64-byte runs of the image (four rows
// of one 4-column group each) and writes four 64-byte runs of bf16 rows, so both sides move whole
// 32-byte sectors; HBM-bound: 512 + 256 bytes per q row.
struct DqConvertParams {
  const float* acc;
  __nv_bfloat16* dq;
  int64_t dq_sb, dq_sh, dq_ss;
  int q_heads, n_q_tiles;
  int d_qk;  // columns of dq
  float scale;
  SplashPeerOutput dq_peer;  // second destination in other ranks' memory (ptrs == nullptr: none)
};

__global__ void __launch_bounds__(256) splash_dq_convert_kernel(const DqConvertParams p) {
  const int64_t tile = blockIdx.x;
  const int qt = (int)(tile % p.n_q_tiles);
  const int64_t bh = tile / p.n_q_tiles;
  const int h = (int)(bh % p.q_heads);
  const int64_t b = bh / p.q_heads;
  const float4* src = reinterpret_cast<const float4*>(p.acc + tile * kDqTileFloats);
  __nv_bfloat16* dst = p.dq + b * p.dq_sb + h * p.dq_sh + (int64_t)qt * kTile * p.dq_ss;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jj = lane & 7, rr = lane >> 3;
  float4 v[16];
#pragma unroll
  for (int it = 0; it < 4; ++it)
#pragma unroll
    for (int jg = 0; jg < 4; ++jg) v[it * 4 + jg] = __ldcs(src + (jg * 8 + jj) * kTile + warp * 16 + it * 4 + rr);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int r = warp * 16 + it * 4 + rr;
#pragma unroll
    for (int jg = 0; jg < 4; ++jg) {
      const float4 x = v[it * 4 + jg];
      uint2 w;
      w.x = pack_bf16(x.x * p.scale, x.y * p.scale);
      w.y = pack_bf16(x.z * p.scale, x.w * p.scale);
      if ((jg * 8 + jj) * 4 < p.d_qk) {
        *reinterpret_cast<uint2*>(dst + (int64_t)r * p.dq_ss + (jg * 8 + jj) * 4) = w;
        if (p.dq_peer.ptrs)
          *reinterpret_cast<uint2*>(peer_row(p.dq_peer, (int)b, h, qt * kTile + r) + (jg * 8 + jj) * 4) = w;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// host launcher
// ------------------------------------------------------------------------------------------
size_t bwd_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len) {
  if (batch <= 0 || q_heads <= 0 || q_len <= 0) return 0;
  const size_t n = (size_t)batch * (size_t)q_heads * (size_t)q_len * sizeof(float);
  return 2 * ((n + 255) & ~(size_t)255);  // di, then -logsumexp * log2(e)
}
// Fused form: the same two per-row arrays, then the fp32 dQ image.
size_t bwd_fused_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len) {
  const size_t base = bwd_workspace_bytes(batch, q_heads, q_len);
  if (base == 0) return 0;
  return base + (size_t)batch * (size_t)q_heads * (size_t)q_len * kHeadDim * sizeof(float);
}

int launch_bwd(const SplashBwdArgs& a, cudaStream_t stream) {
  int st;
  const SplashTensor* ts[8] = {&a.q, &a.k, &a.v, &a.o, &a.d_o, &a.dq, &a.dk, &a.dv};
  for (int i = 0; i < 8; ++i)
    if ((st = check_bf16_tensor(*ts[i]))) return st;
  const int64_t B = a.q.size[0], Hq = a.q.size[1], Sq = a.q.size[2], D = a.q.size[3];
  const int64_t Hkv = a.k.size[1], Skv = a.k.size[2];
  // head dims below 128 are read in place (zero-extended by the TMA boxes), see splash_fwd
  const int64_t Dv = a.v.size[3];
  // head dims above 128 (up to 256): three passes over 128-column panels, splash_bwd_wide_sm100.cu
  if (D > 2 * kHeadDim || Dv > 2 * kHeadDim) return SPLASH_ERR_UNSUPPORTED;
  const bool wide = D > kHeadDim || Dv > kHeadDim;
  if (D % 8 != 0 || Dv % 8 != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  auto same3 = [](const SplashTensor& x, const SplashTensor& y) {
    return x.size[0] == y.size[0] && x.size[1] == y.size[1] && x.size[2] == y.size[2];
  };
  if (!same3(a.q, a.o) || !same3(a.q, a.d_o) || !same3(a.q, a.dq) || !same3(a.k, a.v) || !same3(a.k, a.dk) ||
      !same3(a.k, a.dv) || a.k.size[0] != B || a.k.size[3] != D || a.dq.size[3] != D || a.dk.size[3] != D ||
      a.o.size[3] != Dv || a.d_o.size[3] != Dv || a.dv.size[3] != Dv)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (Hkv <= 0 || Hq % Hkv != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (Sq % kTile != 0 || Skv % kTile != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if ((a.q_segment_ids == nullptr) != (a.kv_segment_ids == nullptr))
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (a.logsumexp == nullptr || a.error_record == nullptr || a.workspace == nullptr)
    return SPLASH_ERR_INVALID_ARGUMENT;
  const bool fused = (a.flags & SPLASH_BWD_FUSED_DQ) != 0 && !wide;  // the wide passes are separate by construction
  if ((st = check_peer_output(a.dq_peer, Sq, D)) || (st = check_peer_output(a.dk_peer, Skv, D)) ||
      (st = check_peer_output(a.dv_peer, Skv, Dv)))
    return st;
  if ((a.dq_peer.ptrs || a.dk_peer.ptrs || a.dv_peer.ptrs) && !fused) return SPLASH_ERR_UNSUPPORTED;
  if (a.workspace_bytes < (fused ? bwd_fused_workspace_bytes(B, Hq, Sq) : bwd_workspace_bytes(B, Hq, Sq)))
    return SPLASH_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a.workspace) & 255u) != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (a.sched_dkv.row_ptr == nullptr || a.sched_dkv.entries == nullptr || a.sched_dkv.n_rows != Skv / kTile)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (!fused && (a.sched_dq.row_ptr == nullptr || a.sched_dq.entries == nullptr || a.sched_dq.n_rows != Sq / kTile))
    return SPLASH_ERR_INVALID_ARGUMENT;  // the fused form walks the dkv schedule only
  if (a.mask_fn.kind == SPLASH_MASK_CHUNKED && a.mask_fn.chunk <= 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (Hq > 65535 || B > 65535 || Sq / kTile > 65535 || Skv / kTile > 65535) return SPLASH_ERR_TOO_LARGE;
  if (!(a.scale > 0.f) || !(a.scale < 1.0e30f)) return SPLASH_ERR_INVALID_ARGUMENT;

  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  if ((st = make_tile_tensor_map(&tm_q, a.q, kTile)) || (st = make_tile_tensor_map(&tm_do, a.d_o, kTile)) ||
      (st = make_tile_tensor_map(&tm_k, a.k, kTile)) || (st = make_tile_tensor_map(&tm_v, a.v, kTile)))
    return st;

  const uint32_t mask = a.launch_mask == 0 ? 7u : a.launch_mask;
  float* delta = static_cast<float*>(a.workspace);
  float* nlse2 = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + bwd_workspace_bytes(B, Hq, Sq) / 2);
  float* dq_acc = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + bwd_workspace_bytes(B, Hq, Sq));
  // (fused form: the image the reds add into starts at zero; the di pass clears it while it streams)
  if (mask & 1u) {
    DeltaParams dp;
    dp.o = static_cast<const __nv_bfloat16*>(a.o.data);
    dp.d_o = static_cast<const __nv_bfloat16*>(a.d_o.data);
    dp.o_sb = a.o.stride[0];
    dp.o_sh = a.o.stride[1];
    dp.o_ss = a.o.stride[2];
    dp.do_sb = a.d_o.stride[0];
    dp.do_sh = a.d_o.stride[1];
    dp.do_ss = a.d_o.stride[2];
    dp.delta = delta;
    dp.lse = a.logsumexp;
    dp.nlse2 = nlse2;
    dp.q_heads = (int)Hq;
    dp.q_len = (int)Sq;
    dp.d_v = (int)Dv;
    dp.n_rows = B * Hq * Sq;
    dp.dq_image = fused ? dq_acc : nullptr;
    const unsigned blocks = (unsigned)((dp.n_rows + kDeltaRowsPerBlock - 1) / kDeltaRowsPerBlock);
    splash_delta_kernel<<<blocks, 256, 0, stream>>>(dp);
    if (cudaGetLastError() != cudaSuccess) return SPLASH_ERR_CUDA;
  }

  const bool soft_cap = a.soft_cap != 0.f;
  if (soft_cap && !(a.soft_cap > 0.f)) return SPLASH_ERR_INVALID_ARGUMENT;
  auto* dq_kernel = soft_cap ? splash_dq_kernel<true> : splash_dq_kernel<false>;
  auto* dkv_kernel = fused ? (soft_cap ? splash_dkv_kernel<true, true> : splash_dkv_kernel<false, true>)
                           : (soft_cap ? splash_dkv_kernel<true, false> : splash_dkv_kernel<false, false>);
  const int dkv_smem = kDkvSmemBytes;
  // function attributes are per device: remember which devices have been set up
  {
    static std::mutex attr_mu;
    static bool attr_done[64][4] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SPLASH_ERR_CUDA;
    std::lock_guard<std::mutex> lock(attr_mu);
    bool& done = attr_done[dev][(soft_cap ? 1 : 0) + (fused ? 2 : 0)];
    if (!done) {
      if (cudaFuncSetAttribute(dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmemBytes) !=
              cudaSuccess ||
          cudaFuncSetAttribute(dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv_smem) != cudaSuccess)
        return SPLASH_ERR_CUDA;
      done = true;
    }
  }

  BwdParams p;
  p.out0_peer = SplashPeerOutput{};
  p.out1_peer = SplashPeerOutput{};
  p.nlse2 = nlse2;
  p.delta = delta;
  p.q_seg = a.q_segment_ids;
  p.kv_seg = a.kv_segment_ids;
  p.q_sequence = a.q_sequence;
  p.fn = a.mask_fn;
  p.q_len = (int)Sq;
  p.kv_len = (int)Skv;
  p.q_heads = (int)Hq;
  p.kv_heads = (int)Hkv;
  p.d_qk = (int)D;
  p.d_v = (int)Dv;
  p.nk_qk = (int)((D + 15) / 16);
  p.nk_v = (int)((Dv + 15) / 16);
  p.scale = a.scale;
  p.scale_log2 = a.scale * kLog2e;
  p.err = a.error_record;
  p.soft_cap = a.soft_cap;
  p.softcap_a = soft_cap ? a.scale / a.soft_cap : 0.f;
  p.dq_acc = fused ? dq_acc : nullptr;
  if (wide) return launch_bwd_wide(tm_q, tm_do, tm_k, tm_v, p, a, soft_cap, mask, stream);

  // dq (split form)
  p.out0 = static_cast<__nv_bfloat16*>(a.dq.data);
  p.out0_sb = a.dq.stride[0];
  p.out0_sh = a.dq.stride[1];
  p.out0_ss = a.dq.stride[2];
  p.out1 = nullptr;
  p.out1_sb = p.out1_sh = p.out1_ss = 0;
  p.row_ptr = a.sched_dq.row_ptr;
  p.entries = reinterpret_cast<const int4*>(a.sched_dq.entries);
  p.row_order = a.sched_dq.row_order;
  p.row_end = a.sched_dq.row_end;
  p.entries_per_batch = a.sched_dq.entries_per_batch;
  p.pmb = a.sched_dq.partial_mask_blocks;
  p.pm_bq = a.sched_dq.block_q > 0 ? a.sched_dq.block_q : kTile;
  p.pm_bkv = a.sched_dq.block_kv > 0 ? a.sched_dq.block_kv : kTile;
  p.n_rows = a.sched_dq.n_rows;
  // dq: the q heads of one kv head stream the same K / V
  p.n_groups = (int)(Hq * B);
  p.chunk_groups = chunk_groups_for(2 * Skv * kHeadDim * 2 / (Hq / Hkv), p.n_groups, Hq / Hkv);
  if ((int64_t)p.n_rows * p.n_groups > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;
  if (!fused && (mask & 2u))
    dq_kernel<<<dim3((unsigned)(p.n_rows * p.n_groups), 1u, 1u), kBwdThreads, kDqSmemBytes, stream>>>(
        tm_q, tm_do, tm_k, tm_v, p);
  if (cudaGetLastError() != cudaSuccess) return SPLASH_ERR_CUDA;

  // dkv
  p.out0 = static_cast<__nv_bfloat16*>(a.dk.data);
  p.out0_sb = a.dk.stride[0];
  p.out0_sh = a.dk.stride[1];
  p.out0_ss = a.dk.stride[2];
  p.out1 = static_cast<__nv_bfloat16*>(a.dv.data);
  p.out1_sb = a.dv.stride[0];
  p.out1_sh = a.dv.stride[1];
  p.out1_ss = a.dv.stride[2];
  p.out0_peer = a.dk_peer;
  p.out1_peer = a.dv_peer;
  p.row_ptr = a.sched_dkv.row_ptr;
  p.entries = reinterpret_cast<const int4*>(a.sched_dkv.entries);
  p.row_order = a.sched_dkv.row_order;
  p.row_end = a.sched_dkv.row_end;
  p.entries_per_batch = a.sched_dkv.entries_per_batch;
  p.pmb = a.sched_dkv.partial_mask_blocks;
  p.pm_bq = a.sched_dkv.block_q > 0 ? a.sched_dkv.block_q : kTile;
  p.pm_bkv = a.sched_dkv.block_kv > 0 ? a.sched_dkv.block_kv : kTile;
  p.n_rows = a.sched_dkv.n_rows;
  // dkv: the kv tiles of one (batch, kv head) stream the same Q / dO of its q-head group
  p.n_groups = (int)(Hkv * B);
  // (fused: plus the fp32 dQ image of those heads, which the reds keep in L2)
  p.chunk_groups = chunk_groups_for((Hq / Hkv) * Sq * kHeadDim * (fused ? 8 : 4), p.n_groups, 1);
  if ((int64_t)p.n_rows * p.n_groups > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;
  if (mask & 4u)
    dkv_kernel<<<dim3((unsigned)(p.n_rows * p.n_groups), 1u, 1u), fused ? kFusedThreads : kDkvThreads, dkv_smem,
                 stream>>>(tm_q, tm_do, tm_k, tm_v, p);
  if (cudaGetLastError() != cudaSuccess) return SPLASH_ERR_CUDA;
  if (fused && (mask & 2u)) {
    DqConvertParams cp;
    cp.acc = dq_acc;
    cp.dq = static_cast<__nv_bfloat16*>(a.dq.data);
    cp.dq_sb = a.dq.stride[0];
    cp.dq_sh = a.dq.stride[1];
    cp.dq_ss = a.dq.stride[2];
    cp.q_heads = (int)Hq;
    cp.n_q_tiles = (int)(Sq / kTile);
    cp.d_qk = (int)D;
    cp.scale = a.scale;
    cp.dq_peer = a.dq_peer;
    const int64_t n_tiles = B * Hq * (Sq / kTile);
    if (n_tiles > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;
    splash_dq_convert_kernel<<<(unsigned)n_tiles, 256, 0, stream>>>(cp);
  }
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------
// backward with the scratch held in the library image (no allocation anywhere on the path)
// ------------------------------------------------------------------------------------------
// di rows followed by -logsumexp*log2(e) rows, SPLASH_STATIC_SCRATCH_MAX_ROWS each.
static __device__ __align__(256) float g_static_scratch[2 * SPLASH_STATIC_SCRATCH_MAX_ROWS];

int launch_bwd_static_scratch(const SplashBwdArgs& a, cudaStream_t stream) {
  const int64_t B = a.q.size[0], Hq = a.q.size[1], Sq = a.q.size[2];
  if (B <= 0 || Hq <= 0 || Sq <= 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (B * Hq * Sq > (int64_t)SPLASH_STATIC_SCRATCH_MAX_ROWS) return SPLASH_ERR_TOO_LARGE;

  // Inside host code the array's name is only a handle for the runtime, not a device address;
  // the address is looked up once per device, with that device current.
  constexpr int kMaxDevices = 64;
  static float* device_ptr[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SPLASH_ERR_CUDA;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (device_ptr[dev] == nullptr) {
      void* sym = nullptr;
      if (cudaGetSymbolAddress(&sym, g_static_scratch) != cudaSuccess || sym == nullptr) return SPLASH_ERR_CUDA;
      device_ptr[dev] = static_cast<float*>(sym);
    }
    scratch = device_ptr[dev];
  }
  SplashBwdArgs b = a;
  b.flags &= ~(uint32_t)SPLASH_BWD_FUSED_DQ;  // the array holds the two per-row terms only
  b.workspace = scratch;
  b.workspace_bytes = bwd_workspace_bytes(B, Hq, Sq);  // <= sizeof(g_static_scratch) by the row check
  return launch_bwd(b, stream);
}

}  // namespace sb
