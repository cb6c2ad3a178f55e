// Sequence-shard <-> head-shard exchange by peer stores (the Ulysses all-to-all without a
// collective library): every rank copies its outgoing slabs straight into the other ranks' receive
// buffers, which are laid out the way the attention kernels read them, so nothing is packed before
// or unpacked after the transfer.
//
// The reference has no all-to-all (its context-parallel wrapper is ring attention over
// lax.ppermute, ring_attention_kernel.py:95-99); this stands where `jax.lax.all_to_all(x, axis,
// split_axis=heads, concat_axis=seq)` would around the kernels.
//
// Plain 16-byte loads from local memory and 16-byte stores to peer memory only: no TMA, no
// multicast, no multimem.  Ordering between ranks (receive buffers free before the push, all pushes
// landed after it) is the caller's, with two barriers around the call.
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/splash_b200.h"

namespace sb {

struct ExchangeParams {
  const uint8_t* src;
  uint8_t* const* dst_ptrs;
  int world, rank, seq_to_head;
  int64_t batch, h_loc, s_loc;
  int64_t dst_base_bytes;  // where the receive buffer starts inside every rank's mapped block
  int64_t row_bytes;    // head_dim * element size
  int64_t slab_bytes;   // s_loc * row_bytes: one (peer, batch, head) slab, contiguous on both sides
  int chunks_per_slab;
};

constexpr int kExchangeThreads = 256;
constexpr int64_t kExchangeChunk = 64 * 1024;  // bytes one CTA moves: 16 x 16 bytes per thread

__global__ void __launch_bounds__(kExchangeThreads) splash_exchange_push_kernel(const ExchangeParams p) {
  // blockIdx.x = chunk within the slab, blockIdx.y = slab; slabs are numbered peer-fastest and the
  // peer order starts after this rank, so concurrently running CTAs spread over all links
  const int64_t slab = blockIdx.y;
  const int step = (int)(slab % p.world);
  const int64_t bh = slab / p.world;
  const int peer = (p.rank + 1 + step) % p.world;
  const int64_t h = bh % p.h_loc, b = bh / p.h_loc;
  const int64_t heads_all = p.h_loc * p.world, s_all = p.s_loc * p.world;
  int64_t src_off, dst_off;
  if (p.seq_to_head) {  // [B, H, s_loc, D] -> peer's [B, h_loc, S, D]
    src_off = ((b * heads_all + (int64_t)peer * p.h_loc + h) * p.s_loc) * p.row_bytes;
    dst_off = ((b * p.h_loc + h) * s_all + (int64_t)p.rank * p.s_loc) * p.row_bytes;
  } else {              // [B, h_loc, S, D] -> peer's [B, H, s_loc, D]
    src_off = ((b * p.h_loc + h) * s_all + (int64_t)peer * p.s_loc) * p.row_bytes;
    dst_off = ((b * heads_all + (int64_t)p.rank * p.h_loc + h) * p.s_loc) * p.row_bytes;
  }
  const int64_t begin = (int64_t)blockIdx.x * kExchangeChunk;
  const int64_t end = begin + kExchangeChunk < p.slab_bytes ? begin + kExchangeChunk : p.slab_bytes;
  const uint4* src = reinterpret_cast<const uint4*>(p.src + src_off);
  uint4* dst = reinterpret_cast<uint4*>(p.dst_ptrs[peer] + p.dst_base_bytes + dst_off);
  const int64_t i0 = begin / 16 + threadIdx.x, i1 = end / 16;
  uint4 v[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const int64_t i = i0 + (int64_t)k * kExchangeThreads;
    if (i < i1) v[k] = __ldg(src + i);
  }
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const int64_t i = i0 + (int64_t)k * kExchangeThreads;
    if (i < i1) dst[i] = v[k];
  }
}

}  // namespace sb

extern "C" int splash_exchange_push(const SplashExchangeArgs* a, void* cuda_stream) {
  if (a == nullptr || a->src == nullptr || a->dst_ptrs == nullptr) return SPLASH_ERR_INVALID_ARGUMENT;
  if (a->world < 1 || a->rank < 0 || a->rank >= a->world) return SPLASH_ERR_INVALID_ARGUMENT;
  if (a->batch <= 0 || a->h_loc <= 0 || a->s_loc <= 0 || a->row_bytes <= 0 || a->row_bytes % 16 != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a->src) & 15u) != 0 || a->dst_base_bytes < 0 || a->dst_base_bytes % 16 != 0)
    return SPLASH_ERR_INVALID_ARGUMENT;
  sb::ExchangeParams p;
  p.src = static_cast<const uint8_t*>(a->src);
  p.dst_ptrs = reinterpret_cast<uint8_t* const*>(a->dst_ptrs);
  p.world = a->world;
  p.rank = a->rank;
  p.seq_to_head = a->seq_to_head != 0;
  p.batch = a->batch;
  p.h_loc = a->h_loc;
  p.s_loc = a->s_loc;
  p.row_bytes = a->row_bytes;
  p.dst_base_bytes = a->dst_base_bytes;
  p.slab_bytes = a->s_loc * a->row_bytes;
  const int64_t chunks = (p.slab_bytes + sb::kExchangeChunk - 1) / sb::kExchangeChunk;
  const int64_t slabs = (int64_t)a->world * a->batch * a->h_loc;
  if (chunks > 0x7fffffffll || slabs > 65535) return SPLASH_ERR_TOO_LARGE;
  p.chunks_per_slab = (int)chunks;
  sb::splash_exchange_push_kernel<<<dim3((unsigned)chunks, (unsigned)slabs, 1u), sb::kExchangeThreads, 0,
                                    static_cast<cudaStream_t>(cuda_stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? SPLASH_OK : SPLASH_ERR_CUDA;
}
