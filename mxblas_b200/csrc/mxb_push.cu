// mxb_push_block: copy a 2-D block of this GPU's memory into the same position of up to 7 other
// buffers, which may be peer GPUs' memory mapped into this process (symmetric memory / peer access).
//
// It is the exchange step of an N-sharded run that wants the full result on every rank without a
// collective: after its GEMM each rank pushes its column block of the result into every rank's copy.
// The stores go over NVLink as packets, so they are issued as 16 bytes per lane with consecutive lanes
// on consecutive addresses of a row (a warp writes 512 contiguous bytes); the block lands at its place in
// the row-major result, so no re-layout copy follows. The reference is single-GPU and has no counterpart.
//
// (Storing to the peers from the GEMM's own epilogue was tried first: the extra code in the output stage
// cost the single-GPU kernels registers even when nothing was replicated, c3 +35 %, and a thread that owns
// one output row can only send 16- to 64-byte packets.)
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mxblas_b200.h"

namespace {

struct PushDst {
  void* ptr[7];
  int n;
};

// rows x row_bytes (a multiple of 16) from src (pitch src_pitch) to every dst (pitch dst_pitch)
__global__ void __launch_bounds__(256) push_block_kernel(const uint8_t* __restrict__ src, long long src_pitch,
                                                         PushDst dst, long long dst_pitch, long long rows,
                                                         int vec_per_row) {
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    const uint4 val = *reinterpret_cast<const uint4*>(src + r * src_pitch + static_cast<long long>(v) * 16);
    for (int d = 0; d < dst.n; ++d)
      *reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst.ptr[d]) + r * dst_pitch + static_cast<long long>(v) * 16) = val;
  }
}

}  // namespace

extern "C" int mxb_push_block_ex(const void* src, long long src_pitch, void* const* dsts, int copies,
                                 long long dst_pitch, long long rows, long long row_bytes, int max_blocks,
                                 void* stream) {
  if (src == nullptr || dsts == nullptr || copies < 0 || copies > 7 || rows < 0 || row_bytes < 0) return MXB_ERR_INVALID;
  if (copies == 0 || rows == 0 || row_bytes == 0) return MXB_OK;
  if (row_bytes % 16 || src_pitch % 16 || dst_pitch % 16 || (reinterpret_cast<uintptr_t>(src) & 15))
    return MXB_ERR_UNSUPPORTED;
  if (src_pitch < row_bytes || dst_pitch < row_bytes) return MXB_ERR_INVALID;
  PushDst d;
  d.n = copies;
  for (int i = 0; i < 7; ++i) d.ptr[i] = nullptr;
  for (int i = 0; i < copies; ++i) {
    if (dsts[i] == nullptr) return MXB_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(dsts[i]) & 15) return MXB_ERR_UNSUPPORTED;
    d.ptr[i] = dsts[i];
  }
  const long long vec_per_row = row_bytes / 16;
  if (vec_per_row > 0x7fffffffll) return MXB_ERR_UNSUPPORTED;
  const long long total = rows * vec_per_row;
  long long blocks = (total + 255) / 256;
  if (max_blocks <= 0) max_blocks = 148 * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  push_block_kernel<<<static_cast<unsigned int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), src_pitch, d, dst_pitch, rows, static_cast<int>(vec_per_row));
  return cudaGetLastError() == cudaSuccess ? MXB_OK : MXB_ERR_CUDA;
}

extern "C" int mxb_push_block(const void* src, long long src_pitch, void* const* dsts, int copies,
                              long long dst_pitch, long long rows, long long row_bytes, void* stream) {
  return mxb_push_block_ex(src, src_pitch, dsts, copies, dst_pitch, rows, row_bytes, 0, stream);
}

// The same transfer on the copy engines: one 2-D copy per destination. Needs no SM, so it runs beside a
// persistent GEMM that occupies all of them.
extern "C" int mxb_push_block_dma(const void* src, long long src_pitch, void* const* dsts, int copies,
                                  long long dst_pitch, long long rows, long long row_bytes, void* stream) {
  if (src == nullptr || dsts == nullptr || copies < 0 || copies > 7 || rows < 0 || row_bytes < 0) return MXB_ERR_INVALID;
  if (copies == 0 || rows == 0 || row_bytes == 0) return MXB_OK;
  if (src_pitch < row_bytes || dst_pitch < row_bytes) return MXB_ERR_INVALID;
  for (int i = 0; i < copies; ++i) {
    if (dsts[i] == nullptr) return MXB_ERR_INVALID;
    cudaError_t e = cudaMemcpy2DAsync(dsts[i], static_cast<size_t>(dst_pitch), src, static_cast<size_t>(src_pitch),
                                      static_cast<size_t>(row_bytes), static_cast<size_t>(rows),
                                      cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return MXB_ERR_CUDA;
  }
  return MXB_OK;
}
