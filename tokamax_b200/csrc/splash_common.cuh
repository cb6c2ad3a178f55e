// Definitions shared by the forward / dq / dkv kernels and their host launchers.
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through the runtime)
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>

#include "../../include/splash_b200.h"
#include "sm100_ptx.cuh"

namespace sb {

constexpr int kTile = 128;          // q and kv tile edge the MMAs work on
constexpr int kHeadDim = 128;       // head dimension of the bf16 kernels
constexpr int kTileBytes = kTile * kHeadDim * 2;   // one bf16 operand tile: 32 KiB
constexpr int kHalfBytes = kTileBytes / 2;         // one 64-column (128-byte) swizzle half
constexpr float kMaskedLogit = -1.0e30f;           // raw logit given to masked positions
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Per-row key interval kept by an in-kernel mask function (see SplashMaskFn).
struct RowInterval {
  int lo, hi;
};

__device__ __forceinline__ RowInterval mask_fn_interval(const SplashMaskFn& fn, int qi) {
  RowInterval iv;
  iv.lo = INT32_MIN;
  iv.hi = INT32_MAX;
  if (fn.kind == SPLASH_MASK_CAUSAL) {
    iv.hi = qi + fn.offset;
  } else if (fn.kind == SPLASH_MASK_LOCAL) {
    if (fn.has_left) iv.lo = qi + fn.offset - fn.left;
    if (fn.has_right) iv.hi = qi + fn.offset + fn.right;
  } else if (fn.kind == SPLASH_MASK_CHUNKED) {
    iv.lo = (qi / fn.chunk) * fn.chunk;
    iv.hi = qi;
  }
  return iv;
}

// Same mask function seen from a key: the queries i that keep key j form an interval too, but
// the dkv kernel simply evaluates lo(i) <= j <= hi(i) per element, so no inverse is needed.

// Host-side helpers (defined in splash_host.cu).
int make_tile_tensor_map(CUtensorMap* out, const SplashTensor& t, int box_rows);
int check_bf16_tensor(const SplashTensor& t);
int check_e4m3_tensor(const SplashTensor& t);

}  // namespace sb
