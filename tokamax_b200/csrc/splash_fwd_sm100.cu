// Splash attention forward for sm_100a: bf16 (or block-scaled e4m3) Q/K/V, head_dim 128, fp32
// accumulation.
//
// One CTA owns two adjacent 128-row q tiles of one (batch, q head) and walks the kv tiles its
// schedule row lists.  Roles (384 threads):
//   warps 0-3 / 4-7 : softmax warpgroup of q tile 0 / 1 — one thread per score row
//   warp 8          : TMA producer (Q once, then a 4-slot ring of K and V tiles)
//   warp 9          : tcgen05 MMA issuer (and TMEM allocator)
//   warps 10-11     : idle; they complete the third warpgroup so registers can be handed
//                     from it to the softmax warpgroups (setmaxnreg)
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  P (bf16, two values per
// column) overwrites the first 64 columns of its S tile and feeds the PV MMA straight from TMEM.
// The two tiles ping-pong: while the softmax of tile 0 runs on the SIMT lanes, the tensor core
// computes QK^T of tile 1 and PV of the previous step.
//
// Online softmax keeps a possibly stale running maximum: O and l are rescaled only when the
// new row maximum exceeds the one in use by more than 2^8, which keeps the TMEM round trip of
// O off the common path.  logsumexp is exact regardless (it is formed from the maximum in use
// and the matching l).
//
// Follows the arithmetic of the reference forward kernel
// (tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_kernel.py:299-527,
// masking :202-296) with the softmax scale applied in fp32 inside the kernel.
//
// kFp8 = true is the e4m3 prefill variant: Q, K and V hold e4m3 values with one fp32 scale per
// (batch, head, 128-token tile).  Tiles are 128 x 128 bytes (one swizzle atom wide), both MMAs run
// as kind::f8f6f4 with K = 32 per instruction, the product of the q and k tile scales is folded
// into the fp32 softmax scale of each score tile, and P is written back as e4m3 (four values per
// TMEM column) after being multiplied by 2^kFp8PShift and by the V tile's scale relative to the
// largest V scale of the (batch, kv head), so that it sits in the normal range of the format and
// never exceeds it.  There is no counterpart of this variant in the reference, which accepts
// bf16 / f32 only.
#include <mutex>

#include "splash_common.cuh"
#include "splash_fwd_params.cuh"

namespace sb {

struct FwdBarriers {
  uint64_t q_full[2];
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];
  uint64_t s_full[2];
  uint64_t p_half[2];    // the first 64 key columns of P are in TMEM (the first half of the p v MMAs may go)
  uint64_t p_full[2];
  uint64_t o_done[2];
  uint64_t vc_full[2];   // e4m3 with f16 P: a V tile has been converted to f16
  uint64_t vc_empty[2];  //                  the p v MMAs that read it have completed
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t early_exit;
};

constexpr int fwd_smem_bytes(bool fp8, bool p16 = false) {
  return (2 + kFwdStages) * (fp8 ? kFp8TileBytes : kTileBytes) + (p16 ? 2 * kTileBytes : 0) /*f16 V tiles*/ +
         1024 /*barriers*/ + 1024 /*alignment slack*/;
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}\n"
      : "=r"(r)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// four e4m3 values (one 32-bit word, lowest byte first) -> four f16 values, exactly
__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t in, uint32_t& out01, uint32_t& out23) {
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}\n"
      : "=r"(out01), "=r"(out23)
      : "r"(in));
}

// kFp8: e4m3 q / k / v with one scale per 128-token tile.  kP16 (with kFp8): the probabilities stay
// 16 bits wide — q k^T runs on the e4m3 tiles as they are, each V tile is converted once to f16 in
// shared memory (exact: e4m3 values are f16 values) by the two otherwise idle warps, and p v runs as
// an f16 MMA.  That variant meets the bf16 kernel's output bound; the all-e4m3 one does not (P
// rounded to 3 mantissa bits) but spends half the tensor time on p v.
template <bool kFp8, bool kSoftCap, bool kP16 = false>
__global__ void __launch_bounds__(kFwdThreads, 1)
splash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  constexpr int kTB = kFp8 ? kFp8TileBytes : kTileBytes;  // bytes of one operand tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;                                  // 2 tiles
  static_assert(!kP16 || kFp8, "the f16-P variant is a variant of the e4m3 forward");
  uint8_t* kv_smem = smem + 2 * kTB;                       // ring
  uint8_t* vc_smem = smem + (2 + kFwdStages) * kTB;        // kP16: two f16 images of V tiles
  FwdBarriers* bars = reinterpret_cast<FwdBarriers*>(smem + (2 + kFwdStages) * kTB + (kP16 ? 2 * kTileBytes : 0));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const CtaWork work = cta_work(p.row_order, p.n_rows, p.n_groups, p.chunk_groups, true);
  const int row = work.row;
  const int head = work.group % p.q_heads;
  const int batch = work.group / p.q_heads;
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int ebeg = p.row_ptr[row];
  const int eend = p.row_end ? p.row_end[(int64_t)batch * p.n_rows + row] : p.row_ptr[row + 1];
  const int4* entries = p.entries + (int64_t)batch * p.entries_per_batch;
  const int qt0 = row * 2;

  if (threadIdx.x == 0) {
    bars->early_exit = *reinterpret_cast<volatile uint32_t*>(p.err);
    bars->abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->q_full[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_half[i], 4);  // one arrival per softmax warp
      mbar_init(&bars->p_full[i], 4);
      mbar_init(&bars->o_done[i], 1);
      mbar_init(&bars->vc_full[i], 2);   // one arrival per converting warp
      mbar_init(&bars->vc_empty[i], 1);
    }
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      // K tiles sit in the even slots and are released by the MMAs that read them; V tiles sit in the
      // odd slots and, in the f16-P variant, are released by the two warps that convert them
      mbar_init(&bars->kv_empty[s], (kP16 && (s & 1)) ? 2 : 1);
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

  if (warp >= 8) {
   setmaxnreg_dec<kIssueRegs>();
   if (warp >= 10) {
    // Without kP16 these two warps are idle: only there to complete the third warpgroup for the
    // register hand-over.  With it they turn each e4m3 V tile (128 kv rows x 128 bytes, 16-byte
    // chunks swizzled by row & 7 as TMA wrote them) into the f16 tile the p v MMA reads MN-major:
    // two halves of 64 columns, rows of 128 bytes, the same swizzle — the layout a bf16 V tile has.
    if constexpr (kP16) {
      static_assert(kFwdStages % 2 == 0, "V tiles must keep to the odd ring slots");
      const int t = (warp - 10) * 32 + lane;
      uint32_t n = 0;
      for (int e = ebeg; e < eend; ++e, ++n) {
        const uint32_t it = 2 * n + 1, s = it % kFwdStages, j = n & 1u;
        bool ok = mbar_wait(&bars->kv_full[s], (it / kFwdStages) & 1u, ab, 0x600u + s);
        if (ok) ok = mbar_wait(&bars->vc_empty[j], ((n >> 1) & 1u) ^ 1u, ab, 0x610u + j);
        if (!__all_sync(0xffffffffu, ok)) break;
        const uint8_t* raw = kv_smem + s * kTB;
        uint8_t* dst = vc_smem + j * kTileBytes;
#pragma unroll 4
        for (int idx = t; idx < kTile * 8; idx += 64) {
          const int row = idx >> 3, c = idx & 7, x = row & 7;
          const uint4 in = *reinterpret_cast<const uint4*>(raw + row * 128 + ((c ^ x) << 4));
          uint4 lo, hi;
          e4m3x4_to_f16x4(in.x, lo.x, lo.y);
          e4m3x4_to_f16x4(in.y, lo.z, lo.w);
          e4m3x4_to_f16x4(in.z, hi.x, hi.y);
          e4m3x4_to_f16x4(in.w, hi.z, hi.w);
          uint8_t* base = dst + (c >> 2) * kHalfBytes + row * 128;
          const int c2 = (c & 3) * 2;
          *reinterpret_cast<uint4*>(base + ((c2 ^ x) << 4)) = lo;
          *reinterpret_cast<uint4*>(base + (((c2 + 1) ^ x) << 4)) = hi;
        }
        fence_proxy_async_smem();  // the MMA reads shared memory through the async proxy
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->vc_full[j]);
          mbar_arrive(&bars->kv_empty[s]);
        }
      }
    }
   } else if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      for (int i = 0; i < 2; ++i) {
        if (qt0 + i < p.n_q_tiles) {
          uint8_t* dst = q_smem + i * kTB;
          const bool two = !kFp8 && p.d_qk > 64;  // bf16 tiles are two 64-column halves
          mbar_arrive_expect_tx(&bars->q_full[i], (kFp8 || two) ? kTB : kHalfBytes);
          tma_load_4d(dst, &tm_q, &bars->q_full[i], 0, (qt0 + i) * kTile, head, batch);
          if (two) tma_load_4d(dst + kHalfBytes, &tm_q, &bars->q_full[i], 64, (qt0 + i) * kTile, head, batch);
        }
      }
      uint32_t it = 0;
      bool ok = true;
      for (int e = ebeg; e < eend && ok; ++e) {
        const int col = entries[e].x;
        for (int kv = 0; kv < 2 && ok; ++kv, ++it) {
          const uint32_t s = it % kFwdStages;
          const uint32_t ph = (it / kFwdStages) & 1u;
          ok = mbar_wait(&bars->kv_empty[s], ph ^ 1u, ab, 0x100u + s);
          if (!ok) break;
          uint8_t* dst = kv_smem + s * kTB;
          const CUtensorMap* tm = kv == 0 ? &tm_k : &tm_v;
          const bool two = !kFp8 && (kv == 0 ? p.d_qk : p.d_v) > 64;
          mbar_arrive_expect_tx(&bars->kv_full[s], (kFp8 || two) ? kTB : kHalfBytes);
          tma_load_4d(dst, tm, &bars->kv_full[s], 0, col * kTile, kv_head, batch);
          if (two) tma_load_4d(dst + kHalfBytes, tm, &bars->kv_full[s], 64, col * kTile, kv_head, batch);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk =
          kFp8 ? make_idesc_e4m3(kTile, kTile, false, false) : make_idesc_bf16(kTile, kTile, false, false);
      // N of p v: the output's columns — 128, or 64 when v has at most 64 (half the MMA work; the
      // V tile's second half is then neither loaded nor read)
      const int n_pv = (!kFp8 && p.d_v <= 64) ? 64 : kHeadDim;
      // (kind::f16 with format code 0 for A and B is f16 x f16: the same bits as the e4m3 descriptor)
      const uint32_t idesc_pv = kFp8 ? make_idesc_e4m3(kTile, kHeadDim, false, true)
                                     : make_idesc_bf16(kTile, n_pv, false, true);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t vc_addr = smem_u32(vc_smem);
      const uint32_t kv_addr = smem_u32(kv_smem);
      bool ok = true;
      for (int i = 0; i < 2 && ok; ++i)
        if (qt0 + i < p.n_q_tiles) ok = mbar_wait(&bars->q_full[i], 0, ab, 0x200u + i);

      // S_i = Q_i K^T : both operands K-major.  bf16: eight K=16 slices across two swizzle
      // halves; e4m3: four K=32 slices inside the single 128-byte-wide tile.
      auto issue_qk = [&](int i, uint32_t slot) {
        const uint32_t a0 = q_addr + i * kTB;
        const uint32_t b0 = kv_addr + slot * kTB;
        const SmemDesc da = make_smem_desc_sw128(a0, 16, 1024), db = make_smem_desc_sw128(b0, 16, 1024);
        if constexpr (kFp8) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss_f8(tmem + i * kTile, desc_at(da, k * 32), desc_at(db, k * 32), idesc_qk, k > 0 ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            // head dims below 128: the remaining slices multiply zeros (nk_qk == 8 is tested first so
            // that the full-width path stays a straight run of eight MMAs)
            if (p.nk_qk != 8 && k >= p.nk_qk) break;
            const uint32_t off = (k >> 2) * kHalfBytes + (k & 3) * 32;
            umma_ss(tmem + i * kTile, desc_at(da, off), desc_at(db, off), idesc_qk, k > 0 ? 1u : 0u);
          }
        }
        tc_commit(&bars->s_full[i]);
      };
      // O_i (+)= P_i V : A from TMEM, B = V tile read MN-major (head_dim contiguous):
      // 8 kv rows x 128 B per core group (SBO 1024).  bf16: 64-column halves 16 KiB apart (LBO),
      // K=16 slices 2 KiB apart; e4m3: the 128 columns fit one 128-byte row, K=32 slices 4 KiB
      // apart, P packed four values per TMEM column.
      // `half` 0 / 1: the K slices over the first / last 64 key columns of P (the softmax warps hand
      // P over in two halves, so that the first MMAs run while the second half is still being made)
      auto issue_pv = [&](int i, uint32_t slot, bool acc, int half) {
        const uint32_t b0 = kP16 ? vc_addr + slot * kTileBytes : kv_addr + slot * kTB;
        if constexpr (kFp8 && !kP16) {
          const SmemDesc db = make_smem_desc_sw128(b0, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            const int k = half * 2 + kk;
            umma_ts_f8(tmem + 2 * kTile + i * kTile, tmem + i * kTile + k * 8, desc_at(db, k * 4096), idesc_pv,
                       (acc || k > 0) ? 1u : 0u);
          }
        } else {
          const SmemDesc db = make_smem_desc_sw128(b0, kHalfBytes, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const int k = half * 4 + kk;
            umma_ts(tmem + 2 * kTile + i * kTile, tmem + i * kTile + k * 8, desc_at(db, k * 2048), idesc_pv,
                    (acc || k > 0) ? 1u : 0u);
          }
        }
      };

      const int n_ent = eend - ebeg;
      uint32_t pcnt[2] = {0, 0};
      bool started[2] = {false, false};
      if (n_ent > 0 && ok) {
        const int4 e0 = entries[ebeg];
        ok = mbar_wait(&bars->kv_full[0], 0, ab, 0x300u);
        if (ok) {
          mma_issue_fence();
          for (int i = 0; i < 2; ++i)
            if ((e0.y >> (2 * i)) & 3) issue_qk(i, 0);
          tc_commit(&bars->kv_empty[0]);
        }
        int4 nxt = e0;
        for (int n = 0; n < n_ent && ok; ++n) {
          const int4 cur = nxt;
          const bool has_next = n + 1 < n_ent;
          if (has_next) nxt = entries[ebeg + n + 1];
          const uint32_t itv = 2 * n + 1, itk = 2 * n + 2;
          const uint32_t vslot = itv % kFwdStages, kslot = itk % kFwdStages;
          const uint32_t vc = n & 1u;  // kP16: which f16 image holds this step's V
          if constexpr (kP16)
            ok = mbar_wait(&bars->vc_full[vc], (n >> 1) & 1u, ab, 0x340u + vc);
          else
            ok = mbar_wait(&bars->kv_full[vslot], (itv / kFwdStages) & 1u, ab, 0x310u + vslot);
          if (ok && has_next)
            ok = mbar_wait(&bars->kv_full[kslot], (itk / kFwdStages) & 1u, ab, 0x320u + kslot);
          if (!ok) break;
          mma_issue_fence();
          for (int i = 0; i < 2 && ok; ++i) {
            if ((cur.y >> (2 * i)) & 3) {
              ok = mbar_wait(&bars->p_half[i], pcnt[i] & 1u, ab, 0x350u + i);
              if (!ok) break;
              mma_issue_fence();
              issue_pv(i, kP16 ? vc : vslot, started[i], 0);
              ok = mbar_wait(&bars->p_full[i], pcnt[i] & 1u, ab, 0x330u + i);
              if (!ok) break;
              ++pcnt[i];
              mma_issue_fence();
              issue_pv(i, kP16 ? vc : vslot, true, 1);
              started[i] = true;
            }
            if (i == 1) tc_commit(kP16 ? &bars->vc_empty[vc] : &bars->kv_empty[vslot]);
            if (has_next && ((nxt.y >> (2 * i)) & 3)) issue_qk(i, kslot);
          }
          if (ok && has_next) tc_commit(&bars->kv_empty[kslot]);
        }
      }
      tc_commit(&bars->o_done[0]);
      tc_commit(&bars->o_done[1]);
    }
   }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    setmaxnreg_inc<kSoftmaxRegs>();
    const int i = warp >> 2;           // q tile within the pair
    const int wq = warp & 3;           // TMEM lane quarter this warp may touch
    const int r = wq * 32 + lane;      // row within the tile
    const int q_tile = qt0 + i;
    const bool valid = q_tile < p.n_q_tiles;
    const int q_row = valid ? q_tile * kTile + r : 0;
    const int qi = p.q_sequence ? p.q_sequence[q_row] : q_row;
    const RowInterval iv = mask_fn_interval(p.fn, qi);
    const bool has_seg = p.q_seg != nullptr;
    const int q_seg = has_seg ? p.q_seg[(int64_t)batch * p.q_len + q_row] : 0;
    const int32_t* kv_seg_row = has_seg ? p.kv_seg + (int64_t)batch * p.kv_len : nullptr;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const uint32_t t_s = tmem + lane_addr + i * kTile;
    const uint32_t t_o = tmem + lane_addr + 2 * kTile + i * kTile;
    // e4m3: scores carry the q tile's and the kv tile's scale; V tiles are weighted relative to
    // the largest V scale of this (batch, kv head).
    float cq = kSoftCap ? p.soft_cap * kLog2e : p.scale_log2;  // score -> log2 units
    float v_ref = 1.f;
    const float* k_scale = nullptr;
    const float* v_scale = nullptr;
    if constexpr (kFp8) {
      const int64_t kbase = ((int64_t)batch * p.kv_heads + kv_head) * p.n_kv_tiles;
      k_scale = p.k_scale + kbase;
      v_scale = p.v_scale + kbase;
      if (valid) cq *= p.q_scale[((int64_t)batch * p.q_heads + head) * p.n_q_tiles + q_tile];
      float vm = 0.f;
      for (int t = lane; t < p.n_kv_tiles; t += 32) vm = fmaxf(vm, __ldg(v_scale + t));
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, off));
      v_ref = vm > 0.f ? vm : 1.f;
    }
    // e4m3 P must stay below 448; f16 P (times 2^6) below 65504; bf16 P has the range of fp32
    constexpr float kThreshold = (kFp8 && !kP16) ? kFp8RescaleThreshold : kRescaleThreshold;

    float m_used = -INFINITY;  // scaled (log2) units
    float m_true = kMaskedLogit;
    float l = 0.f;
    // A sink starts the row as one extra key of weight 1 at the sink logit; a fixed maximum
    // replaces the running one for the whole row (and a sink is then weighed against it).
    const bool fixed_max = p.max_logit_value != nullptr;
    float sink2 = -INFINITY;  // sink logit in log2 units
    if (p.sinks != nullptr) sink2 = p.sinks[head] * kLog2e;
    if (fixed_max) {
      m_used = p.max_logit_value[head] * kLog2e;
      if (p.sinks != nullptr) l = ex2(sink2 - m_used);
    } else if (p.sinks != nullptr) {
      m_used = sink2;
      l = 1.f;
    }
    uint32_t cnt = 0;
    bool started = false;
    bool ok = true;

    int4 ent_next = ebeg < eend ? entries[ebeg] : make_int4(0, 0, 0, 0);
    float ks_next = 1.f, vs_next = 1.f;
    if constexpr (kFp8) {
      if (ebeg < eend) {
        ks_next = __ldg(k_scale + ent_next.x);
        vs_next = __ldg(v_scale + ent_next.x);
      }
    }
    for (int e = ebeg; e < eend; ++e) {
      const int4 ent = ent_next;
      const float ks = ks_next, vs = vs_next;
      if (e + 1 < eend) {  // fetched a step ahead of its use
        ent_next = entries[e + 1];
        if constexpr (kFp8) {
          ks_next = __ldg(k_scale + ent_next.x);
          vs_next = __ldg(v_scale + ent_next.x);
        }
      }
      const float c = fmaxf(kFp8 ? cq * ks : cq, kMinScaleLog2);
      const int st = (ent.y >> (2 * i)) & 3;
      if (st == 0) continue;
      ok = mbar_wait(&bars->s_full[i], cnt & 1u, ab, 0x400u + i);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++cnt;
      tc_fence_after();

      float s[kTile];
      {
        uint32_t v0[32], v1[32], v2[32], v3[32];
        tmem_ld32(t_s, v0);
        tmem_ld32(t_s + 32, v1);
        tmem_ld32(t_s + 64, v2);
        tmem_ld32(t_s + 96, v3);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          s[j] = __uint_as_float(v0[j]);
          s[32 + j] = __uint_as_float(v1[j]);
          s[64 + j] = __uint_as_float(v2[j]);
          s[96 + j] = __uint_as_float(v3[j]);
        }
      }
      if constexpr (kSoftCap) {
        // s <- tanh(scale * s / cap) before masking (reference :202-296 caps, then masks); the
        // factor cap * log2(e) that follows is `c`.
#pragma unroll
        for (int j = 0; j < kTile; ++j) s[j] = tanh_ex2(s[j] * p.softcap_a);
      }
      const int kv0 = ent.x * kTile;
      if (st == 1) {
        if (p.fn.kind != SPLASH_MASK_TABLE) {
          const int lo_rel = iv.lo <= kv0 ? 0 : iv.lo - kv0;
          const int hi_rel = iv.hi >= kv0 + (kTile - 1) ? kTile - 1 : iv.hi - kv0;
#pragma unroll
          for (int j = 0; j < kTile; ++j)
            if (j < lo_rel || j > hi_rel) s[j] = kMaskedLogit;
        } else {
          const int pid = i == 0 ? ent.z : ent.w;
          const int8_t* mrow = p.pmb + ((int64_t)pid * p.pm_bq + (q_row % p.pm_bq)) * p.pm_bkv +
                               (kv0 % p.pm_bkv);
          const int4* m4 = reinterpret_cast<const int4*>(mrow);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
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
        for (int g = 0; g < 32; ++g) {
          const int4 sv = __ldg(sg4 + g);
          if (sv.x != q_seg) s[g * 4 + 0] = kMaskedLogit;
          if (sv.y != q_seg) s[g * 4 + 1] = kMaskedLogit;
          if (sv.z != q_seg) s[g * 4 + 2] = kMaskedLogit;
          if (sv.w != q_seg) s[g * 4 + 3] = kMaskedLogit;
        }
      }

      // The softmax warps are bound by instruction issue, so the per-element work uses the
      // two-wide fp32 instructions of sm_100 (fma / add on register pairs) and three-input max.
      float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
      float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
      for (int j = 12; j < kTile - 4; j += 8) {
        mx0 = max3(mx0, s[j], s[j + 1]);
        mx1 = max3(mx1, s[j + 2], s[j + 3]);
        mx2 = max3(mx2, s[j + 4], s[j + 5]);
        mx3 = max3(mx3, s[j + 6], s[j + 7]);
      }
      mx0 = max3(mx0, s[kTile - 4], s[kTile - 3]);
      mx1 = max3(mx1, s[kTile - 2], s[kTile - 1]);
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(mx * c, kLogitFloor);
      m_true = fmaxf(m_true, kFp8 ? m_new : mx);  // e4m3: log2 units (the scale varies by tile)
      const bool need = !fixed_max && m_new > m_used + kThreshold;
      if (__any_sync(0xffffffffu, need)) {
        const float m_next = fmaxf(m_used, m_new);
        const float alpha = ex2(m_used - m_next);
        l *= alpha;
        if (started) {
          uint32_t v[32];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            tmem_ld32(t_o + g * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
            tmem_st32(t_o + g * 32, v);
          }
        }
        m_used = m_next;
      }

      float ls0 = 0.f, ls1 = 0.f;
      if constexpr (kP16) {
        // as the e4m3 branch below, but P stays 16 bits wide (f16: 11 significant bits; the factor
        // 2^6 keeps the small weights out of the subnormals, 2^(6+8) is the largest value written)
        const float r = fmaxf(__fdividef(vs, v_ref), 5.9604645e-8f);
        const float m_sub = m_used - kFp8PShift - __log2f(r);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float p0 = ex2(fmaf(s[g * 32 + 2 * j], c, -m_sub));
            const float p1 = ex2(fmaf(s[g * 32 + 2 * j + 1], c, -m_sub));
            ls0 += p0;
            ls1 += p1;
            pk[j] = pack_f16(p0, p1);
          }
          tmem_st16(t_s + g * 16, pk);
          if (g == 1) {  // the first 64 key columns are in place
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_half[i]);
          }
        }
        l += (ls0 + ls1) * __fdividef(0.015625f, r);
      } else if constexpr (kFp8) {
        // P * 2^shift * r with r = v scale / largest v scale in (0, 1]; r is floored so that a
        // tile of zeros (scale 0) still counts in l.
        const float r = fmaxf(__fdividef(vs, v_ref), 5.9604645e-8f);
        const float m_sub = m_used - kFp8PShift - __log2f(r);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float p0 = ex2(fmaf(s[g * 64 + 4 * j], c, -m_sub));
            const float p1 = ex2(fmaf(s[g * 64 + 4 * j + 1], c, -m_sub));
            const float p2 = ex2(fmaf(s[g * 64 + 4 * j + 2], c, -m_sub));
            const float p3 = ex2(fmaf(s[g * 64 + 4 * j + 3], c, -m_sub));
            ls0 += p0 + p2;
            ls1 += p1 + p3;
            pk[j] = pack_e4m3x4(p0, p1, p2, p3);
          }
          tmem_st16(t_s + g * 16, pk);
          if (g == 0) {  // the first 64 key columns are in place
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_half[i]);
          }
        }
        l += (ls0 + ls1) * __fdividef(0.015625f, r);  // back to exp2(s - m) units (2^-6 / r)
      } else {
        const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_used, -m_used);
        float2 lsa = make_float2(0.f, 0.f), lsb = make_float2(0.f, 0.f);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
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
          tmem_st16(t_s + g * 16, pk);
          if (g == 1) {  // the first 64 key columns are in place
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_half[i]);
          }
        }
        ls0 = lsa.x + lsb.x;
        ls1 = lsa.y + lsb.y;
        l += ls0 + ls1;
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[i]);
      started = true;
    }

    // ---- epilogue: O / l -> bf16, logsumexp, max_logits
    if (ok) {
      ok = mbar_wait(&bars->o_done[i], 0, ab, 0x500u + i);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && valid) {
      tc_fence_after();
      __nv_bfloat16* orow = p.o + (int64_t)batch * p.o_sb + (int64_t)head * p.o_sh +
                            (int64_t)q_row * p.o_ss;
      uint4* o4 = reinterpret_cast<uint4*>(orow);
      // context parallelism: the row also goes to the rank that owns it in the sequence-sharded layout
      uint4* peer4 = p.o_peer.ptrs ? reinterpret_cast<uint4*>(peer_row(p.o_peer, batch, head, q_row)) : nullptr;
      // e4m3: O accumulated P * 2^shift * (v scale / v_ref) times the stored V values
      const bool live = l > 0.f;  // a row that met a live key, or has a sink
      const float inv = live ? (kFp8 ? v_ref * 0.015625f / l : 1.0f / l) : 0.f;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t v[32];
        if (started) {
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
          if ((g * 4 + j) * 8 < p.d_v) {
            o4[g * 4 + j] = w;
            if (peer4) peer4[g * 4 + j] = w;
          }
        }
      }
      const int64_t stat = ((int64_t)batch * p.q_heads + head) * p.q_len + q_row;
      if (p.lse) p.lse[stat] = live ? (m_used + log2f(l)) * kLn2 : p.mask_value;
      if (p.maxl) {
        float mv = kFp8 ? m_true * kLn2 : m_true * (kSoftCap ? p.soft_cap : p.scale);
        if (p.sinks != nullptr) mv = fmaxf(mv, sink2 * kLn2);
        if (fixed_max) mv = m_used * kLn2;
        p.maxl[stat] = live ? mv : p.mask_value;
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

// ------------------------------------------------------------------------------------------
// host launcher
// ------------------------------------------------------------------------------------------
static int launch_fwd_common(const SplashFwdArgs& a, const float* q_scale, const float* k_scale,
                             const float* v_scale, bool fp8, bool p16, cudaStream_t stream) {
  int st;
  const bool soft_cap = a.soft_cap != 0.f;
  if (soft_cap && (fp8 || !(a.soft_cap > 0.f))) return fp8 ? SPLASH_ERR_UNSUPPORTED : SPLASH_ERR_INVALID_ARGUMENT;
  // a fixed maximum below the true one would push the narrow P formats of the e4m3 forward out of range
  if (fp8 && a.max_logit_value != nullptr) return SPLASH_ERR_UNSUPPORTED;
  if (fp8) {
    if ((st = check_e4m3_tensor(a.q)) || (st = check_e4m3_tensor(a.k)) || (st = check_e4m3_tensor(a.v)))
      return st;
    if (q_scale == nullptr || k_scale == nullptr || v_scale == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  } else {
    if ((st = check_bf16_tensor(a.q)) || (st = check_bf16_tensor(a.k)) || (st = check_bf16_tensor(a.v)))
      return st;
  }
  if ((st = check_bf16_tensor(a.o))) return st;
  if ((st = check_peer_output(a.o_peer, a.q.size[2], a.v.size[3]))) return st;
  if (a.o_peer.ptrs != nullptr && (fp8 || a.q.size[3] > kHeadDim || a.v.size[3] > kHeadDim)) return SPLASH_ERR_UNSUPPORTED;
  const int64_t B = a.q.size[0], Hq = a.q.size[1], Sq = a.q.size[2], D = a.q.size[3];
  const int64_t Hkv = a.k.size[1], Skv = a.k.size[2];
  // Head dims: the MMA tile is 128 wide.  bf16 tensors with fewer columns (a multiple of 8, so rows
  // stay 16-byte aligned) are read in place — the TMA boxes reach past the row's end and the part
  // outside the tensor arrives as zeros, which change neither q k^T nor p v — and only the real
  // columns of the output are stored.  Head dims above 128 (up to 256) go to the forward that works
  // on two 128-column panels (splash_fwd_wide_sm100.cu); e4m3 takes 128 only.
  const int64_t Dv = a.v.size[3];
  constexpr int64_t kMaxWideDim = 2 * kHeadDim;
  if (D > kMaxWideDim || Dv > kMaxWideDim || (fp8 && (D != kHeadDim || Dv != kHeadDim))) return SPLASH_ERR_UNSUPPORTED;
  const bool wide = D > kHeadDim || Dv > kHeadDim;
  if (D % 8 != 0 || Dv % 8 != 0 || a.k.size[3] != D) return SPLASH_ERR_INVALID_ARGUMENT;
  if (a.k.size[0] != B || a.v.size[0] != B || a.o.size[0] != B) return SPLASH_ERR_INVALID_ARGUMENT;
  if (a.v.size[1] != Hkv || a.v.size[2] != Skv || a.o.size[1] != Hq || a.o.size[2] != Sq ||
      a.o.size[3] != Dv)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (Hkv <= 0 || Hq % Hkv != 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if (Sq % kTile != 0 || Skv % kTile != 0 || Sq <= 0 || Skv <= 0) return SPLASH_ERR_INVALID_ARGUMENT;
  if ((a.q_segment_ids == nullptr) != (a.kv_segment_ids == nullptr))
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (a.error_record == nullptr || a.sched.row_ptr == nullptr || a.sched.entries == nullptr)
    return SPLASH_ERR_INVALID_ARGUMENT;
  const int n_q_tiles = (int)(Sq / kTile);
  if (a.sched.n_rows != (n_q_tiles + 1) / 2) return SPLASH_ERR_INVALID_ARGUMENT;
  if (a.mask_fn.kind == SPLASH_MASK_CHUNKED && a.mask_fn.chunk <= 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if (Hq > 65535 || B > 65535 || n_q_tiles > 2 * 65535) return SPLASH_ERR_TOO_LARGE;
  if (!(a.scale > 0.f) || !(a.scale < 1.0e30f)) return SPLASH_ERR_INVALID_ARGUMENT;

  CUtensorMap tm_q, tm_k, tm_v;
  if ((st = make_tile_tensor_map(&tm_q, a.q, kTile)) || (st = make_tile_tensor_map(&tm_k, a.k, kTile)) ||
      (st = make_tile_tensor_map(&tm_v, a.v, kTile)))
    return st;

  FwdParams p;
  p.o = static_cast<__nv_bfloat16*>(a.o.data);
  p.o_sb = a.o.stride[0];
  p.o_sh = a.o.stride[1];
  p.o_ss = a.o.stride[2];
  p.o_peer = a.o_peer;
  p.d_v = (int)Dv;
  p.nk_qk = (int)((D + 15) / 16);
  p.d_qk = (int)D;
  p.lse = a.logsumexp;
  p.maxl = a.max_logits;
  p.q_seg = a.q_segment_ids;
  p.kv_seg = a.kv_segment_ids;
  p.q_sequence = a.q_sequence;
  p.row_ptr = a.sched.row_ptr;
  p.entries = reinterpret_cast<const int4*>(a.sched.entries);
  p.row_order = a.sched.row_order;
  p.row_end = a.sched.row_end;
  p.entries_per_batch = a.sched.entries_per_batch;
  p.pmb = a.sched.partial_mask_blocks;
  p.pm_bq = a.sched.block_q > 0 ? a.sched.block_q : kTile;
  p.pm_bkv = a.sched.block_kv > 0 ? a.sched.block_kv : kTile;
  p.fn = a.mask_fn;
  p.q_len = (int)Sq;
  p.kv_len = (int)Skv;
  p.q_heads = (int)Hq;
  p.kv_heads = (int)Hkv;
  p.n_q_tiles = n_q_tiles;
  p.n_rows = a.sched.n_rows;
  p.scale = a.scale;
  p.scale_log2 = a.scale * kLog2e;
  p.mask_value = a.mask_value;
  p.err = a.error_record;
  p.q_scale = q_scale;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.n_kv_tiles = (int)(Skv / kTile);
  p.sinks = a.sinks;
  p.max_logit_value = a.max_logit_value;
  p.soft_cap = a.soft_cap;
  p.softcap_a = soft_cap ? a.scale / a.soft_cap : 0.f;

  // The q heads of one kv head stream the same K / V (2 tensors of Skv x 128 elements).
  p.n_groups = (int)(Hq * B);
  const int64_t kv_row_bytes = fp8 ? 2 * kHeadDim : 2 * ((D > kHeadDim ? D : kHeadDim) + (Dv > kHeadDim ? Dv : kHeadDim));
  p.chunk_groups = chunk_groups_for(Skv * kv_row_bytes / (Hq / Hkv), p.n_groups, Hq / Hkv);
  if (wide) return launch_fwd_wide(tm_q, tm_k, tm_v, p, soft_cap, stream);
  if ((int64_t)p.n_rows * p.n_groups > 0x7fffffffll) return SPLASH_ERR_TOO_LARGE;
  dim3 grid((unsigned)(p.n_rows * p.n_groups), 1u, 1u);
  // The dynamic shared-memory attribute is per device and per kernel variant: set once, under a
  // lock (calls may come from several threads).
  const int variant = fp8 ? (p16 ? 3 : 1) : (soft_cap ? 2 : 0);
  const int smem = fwd_smem_bytes(fp8, fp8 && p16);
  const void* fn = fp8 ? (p16 ? (const void*)splash_fwd_kernel<true, false, true> : (const void*)splash_fwd_kernel<true, false>)
                       : (soft_cap ? (const void*)splash_fwd_kernel<false, true> : (const void*)splash_fwd_kernel<false, false>);
  {
    static std::mutex attr_mu;
    static bool attr_done[64][4] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SPLASH_ERR_CUDA;
    std::lock_guard<std::mutex> lock(attr_mu);
    if (!attr_done[dev][variant]) {
      if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return SPLASH_ERR_CUDA;
      attr_done[dev][variant] = true;
    }
  }
  if (fp8 && p16)
    splash_fwd_kernel<true, false, true><<<grid, kFwdThreads, smem, stream>>>(tm_q, tm_k, tm_v, p);
  else if (fp8)
    splash_fwd_kernel<true, false><<<grid, kFwdThreads, smem, stream>>>(tm_q, tm_k, tm_v, p);
  else if (soft_cap)
    splash_fwd_kernel<false, true><<<grid, kFwdThreads, smem, stream>>>(tm_q, tm_k, tm_v, p);
  else
    splash_fwd_kernel<false, false><<<grid, kFwdThreads, smem, stream>>>(tm_q, tm_k, tm_v, p);
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}

int launch_fwd(const SplashFwdArgs& a, cudaStream_t stream) {
  return launch_fwd_common(a, nullptr, nullptr, nullptr, false, false, stream);
}

int launch_fwd_fp8(const SplashFwdFp8Args& a, cudaStream_t stream) {
  if (a.flags & ~(uint32_t)SPLASH_FP8_P_F16) return SPLASH_ERR_INVALID_ARGUMENT;
  return launch_fwd_common(a.base, a.q_scale, a.k_scale, a.v_scale, true, (a.flags & SPLASH_FP8_P_F16) != 0, stream);
}

}  // namespace sb
