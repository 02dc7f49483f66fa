// Fully sharded parameters over peer-mapped memory (one node, NVLink / NVSwitch): the stand-alone gather.
//
// Rank r keeps piece r of every unit of the flat parameter space (bf16 parameters in the symmetric heap, where
// peers read them; fp32 master weights and Adam moments privately), concatenated in "shard order".  A layer's
// full bf16 weights exist only in a local staging buffer while the layer runs.  Weight MATRICES are pulled
// from the owners by the GEMM that consumes them (gemm2cta_tcgen05.cu, the gather runs inside that kernel);
// this file holds the plain copy kernel that brings in everything else (biases, LayerNorm parameters,
// embeddings) and serves as the unfused baseline for the matrices:
//
//   fsdp_gather   elements [e0, e1) of a unit -> local staging buffer: element e lives in rank (e / piece_len)'s
//                 shard at shard_off + e % piece_len and is pulled with 16-byte peer loads (every rank reads
//                 1/world of the range from every peer, so all links carry the same load).  No flags are
//                 needed: shards only change inside update_pieces, which every rank enters after all its
//                 gathers of the step, and the step ends with a barrier before the next gathers start.
//
// The gradient side (per-layer reduce-scatter, sharded Adam(W)) is in comm_p2p.cu.  Counterpart of FSDP's
// all-gather in the reference (onmt/train_utils/mp_trainer.py:314-341).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops_api.h"
#include "peer_sync.cuh"

namespace b200 {

__global__ void __launch_bounds__(256)
fsdp_gather_kernel(const NmtgPeerTable t, __nv_bfloat16* __restrict__ dst, long shard_off, long piece_len, long e0, long e1) {
  const long b8 = e0 >> 3, n8 = (e1 - e0) >> 3, p8 = piece_len >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
    // rotate the walk by this rank's piece so that at any moment the peers serve different readers
    const long j = b8 + (i + static_cast<long>(t.rank) * p8) % n8;
    const int owner = static_cast<int>(j / p8);
    const long within = j - owner * p8;
    const uint4 v = reinterpret_cast<const uint4*>(t.works[owner] + shard_off)[within];
    reinterpret_cast<uint4*>(dst)[j] = v;
  }
}

}  // namespace b200

using namespace b200;

const char* nmtg_fsdp_gather(const NmtgPeerTable* t, void* dst, long shard_off, long piece_len, long e0, long e1, int ctas,
                             cudaStream_t stream) {
  if (t->world < 1 || t->world > kMaxRanks) return "fsdp_gather: world size out of range";
  if ((shard_off % 8) || (piece_len % 8) || (e0 % 8) || (e1 % 8) || piece_len <= 0 || e0 < 0 || e1 < e0)
    return "fsdp_gather: offsets must be multiples of 8 elements";
  if (piece_len * t->world < e1) return "fsdp_gather: pieces do not cover the range";
  if (reinterpret_cast<uintptr_t>(dst) & 15) return "fsdp_gather: unaligned staging buffer";
  if (e1 == e0) return nullptr;
  if (ctas < 1) ctas = 32;
  const long need = ((e1 - e0) / 8 + 255) / 256;
  if (need < ctas) ctas = static_cast<int>(need);
  fsdp_gather_kernel<<<ctas, 256, 0, stream>>>(*t, static_cast<__nv_bfloat16*>(dst), shard_off, piece_len, e0, e1);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}
