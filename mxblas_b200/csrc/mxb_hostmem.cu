// mxb_gemm_host: the GEMM for callers whose tensors live in host memory.
//
// The reference has no such path (its operator takes CUDA tensors, mxblas/jit_kernels/mx_gemm.py:340-425);
// a host-resident caller of it pays torch's .cuda() / .cpu() copies around the call. This entry point
// is that whole trip behind one C call: operands go to device staging buffers owned by the library,
// the GEMM runs block by block (row blocks of `left` x column blocks of `right`) so that copies in, GEMMs
// and copies back overlap on three streams, and the call returns when the results are in the caller's
// buffers.
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/mxblas_b200.h"

namespace {

struct Staging {
  void* ptr = nullptr;
  size_t bytes = 0;
};

struct DeviceState {
  Staging left, right, out, ls, rs, os, ws;
  cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
  cudaEvent_t in_ready[16] = {};  // [0..7] row blocks of left, [8..15] column blocks of right
  cudaEvent_t gemm_done[64] = {};
  bool init = false;
};

// one lock per device: calls for different GPUs of one process run side by side, calls for the same GPU
// share its staging buffers and take turns
std::mutex g_mu[64];
DeviceState g_state[64];

// `zero_on` != nullptr: the new buffer is zero-filled on that stream (the GEMMs that read the workspace's
// counters run on it, so the fill is ordered in front of them)
bool ensure(Staging& s, size_t bytes, cudaStream_t zero_on = nullptr) {
  if (bytes == 0) bytes = 256;
  if (s.bytes >= bytes) return true;
  if (s.ptr) cudaFree(s.ptr);
  s.ptr = nullptr;
  s.bytes = 0;
  if (cudaMalloc(&s.ptr, bytes) != cudaSuccess) return false;
  if (zero_on != nullptr && cudaMemsetAsync(s.ptr, 0, bytes, zero_on) != cudaSuccess) return false;
  s.bytes = bytes;
  return true;
}

size_t scale_bytes(int dt) { return dt == MXB_FP32 ? 4 : 2; }

}  // namespace

extern "C" int mxb_gemm_host(const mxb_problem_t* problem, const void* left, const void* right, void* out,
                             const void* left_scale, const void* right_scale, void* out_scale) {
  if (problem == nullptr) return MXB_ERR_INVALID;
  const mxb_problem_t& q = *problem;
  size_t ws_probe = 0;
  int st = mxb_query_workspace(&q, nullptr, &ws_probe);
  if (st != MXB_OK) return st;
  const bool quant = (q.flags & MXB_OUT_QUANT) != 0;
  if (!left || !right || !out || !left_scale || !right_scale || (quant && !out_scale)) return MXB_ERR_INVALID;
  // host tensors must be dense in the layouts the flags name
  const bool out_t = (q.flags & MXB_OUT_TRANSPOSE) != 0;
  const bool cs_t = (q.flags & MXB_OUT_SCALE_TRANSPOSE) != 0;
  const int groups = quant ? q.n / q.qn : 0;
  const int qm = quant && q.qm > 1 ? q.qm : 1;  // rows of the result that share a row of output scales
  if (q.flags & (MXB_LEFT_COL_MAJOR | MXB_RIGHT_ROW_MAJOR)) return MXB_ERR_UNSUPPORTED;  // K-major operands only
  if (q.lda != q.k || q.ldb != q.k) return MXB_ERR_UNSUPPORTED;
  if (q.ldc != (out_t ? q.m : q.n)) return MXB_ERR_UNSUPPORTED;
  if (quant && q.ldcs != (cs_t ? q.m / qm : groups)) return MXB_ERR_UNSUPPORTED;

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return MXB_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_mu[dev]);
  DeviceState& d = g_state[dev];
  if (!d.init) {
    if (cudaStreamCreateWithFlags(&d.h2d, cudaStreamNonBlocking) != cudaSuccess) return MXB_ERR_CUDA;
    if (cudaStreamCreateWithFlags(&d.compute, cudaStreamNonBlocking) != cudaSuccess) return MXB_ERR_CUDA;
    if (cudaStreamCreateWithFlags(&d.d2h, cudaStreamNonBlocking) != cudaSuccess) return MXB_ERR_CUDA;
    for (int i = 0; i < 16; ++i)
      if (cudaEventCreateWithFlags(&d.in_ready[i], cudaEventDisableTiming) != cudaSuccess) return MXB_ERR_CUDA;
    for (int i = 0; i < 64; ++i)
      if (cudaEventCreateWithFlags(&d.gemm_done[i], cudaEventDisableTiming) != cudaSuccess) return MXB_ERR_CUDA;
    d.init = true;
  }

  const size_t esz_out = (q.out_dtype == MXB_E4M3 || q.out_dtype == MXB_E5M2) ? 1 : 2;
  const size_t ssz = scale_bytes(q.scale_dtype);
  const size_t ls_rows = q.m / q.sm, ls_cols = q.k / q.sk;
  const size_t rs_rows = q.n / q.sn;
  // scale strides must describe dense [M/sm, K/sk] (row-major) and dense physical [N/sn, K/sk]
  if (!((q.as_ks == 1 && q.as_rs == static_cast<int64_t>(ls_cols)) || (ls_cols == 1 && ls_rows == 1) ||
        (ls_cols == 1 && q.as_rs == 1)))
    return MXB_ERR_UNSUPPORTED;
  if (!((q.bs_ks == 1 && q.bs_rs == static_cast<int64_t>(ls_cols)) || (ls_cols == 1 && rs_rows == 1) ||
        (ls_cols == 1 && q.bs_rs == 1)))
    return MXB_ERR_UNSUPPORTED;

  // Blocks: `left` in bm row blocks, `right` in bn column blocks (up to 4 x 4) (rows of the physical [N, K] matrix). The
  // host-to-device copies alternate between the two operands, and the GEMM of output block (i, j) starts as
  // soon as row block i and column block j are on the device, so the copy-back of the first blocks runs
  // while most of the operands are still on their way in (PCIe is full duplex). A block holds whole tiles
  // and whole scale and quantisation groups, or lies inside one scale group.
  auto pick = [](int extent, int group, int want, int quantum) {
    int blocks = want;
    while (blocks > 1) {
      const int len = extent / blocks;
      if (extent % blocks == 0 && len % quantum == 0 && (len % group == 0 || group % len == 0)) break;
      blocks /= 2;
    }
    return blocks;
  };
  int bm = 1, bn = 1;
  if (!out_t && !(quant && cs_t)) {
    if (q.m >= 1024) bm = pick(q.m, q.sm, 4, 128);
    if (q.n >= 2048) bn = pick(q.n, q.sn, 4, quant && q.qn > 256 ? q.qn : 256);
    if (quant && bn > 1 && (q.n / bn) % q.qn) bn = 1;
  }
  const int mb = q.m / bm, nb = q.n / bn;

  mxb_problem_t sub = q;
  sub.m = mb;
  sub.n = nb;
  if (q.sm > mb) sub.sm = mb;  // the block lies inside one scale group
  if (q.sn > nb) sub.sn = nb;
  size_t ws_bytes = 0;
  st = mxb_query_workspace(&sub, nullptr, &ws_bytes);
  if (st != MXB_OK) return st;

  if (!ensure(d.left, static_cast<size_t>(q.m) * q.k) || !ensure(d.right, static_cast<size_t>(q.n) * q.k) ||
      !ensure(d.out, static_cast<size_t>(q.m) * q.n * esz_out) || !ensure(d.ls, ls_rows * ls_cols * ssz) ||
      !ensure(d.rs, rs_rows * ls_cols * ssz) ||
      !ensure(d.os, quant ? static_cast<size_t>(q.m / qm) * groups * ssz : 0) || !ensure(d.ws, ws_bytes, d.compute))
    return MXB_ERR_CUDA;

  // every enqueue's return code is kept: the first failure ends the call with MXB_ERR_CUDA after the
  // streams have drained
  cudaError_t first_err = cudaSuccess;
  auto ck = [&](cudaError_t e) {
    if (e != cudaSuccess && first_err == cudaSuccess) first_err = e;
  };

  // scales first (small), then the operand blocks
  ck(cudaMemcpyAsync(d.rs.ptr, right_scale, rs_rows * ls_cols * ssz, cudaMemcpyHostToDevice, d.h2d));
  ck(cudaMemcpyAsync(d.ls.ptr, left_scale, ls_rows * ls_cols * ssz, cudaMemcpyHostToDevice, d.h2d));

  bool launched[8][8] = {};
  int cols_done[8] = {};
  int sent_a = 0, sent_b = 0;
  auto launch_ready = [&]() {
    for (int i = 0; i < sent_a && st == MXB_OK; ++i)
      for (int j = 0; j < sent_b && st == MXB_OK; ++j) {
        if (launched[i][j]) continue;
        launched[i][j] = true;
        const size_t row0 = static_cast<size_t>(i) * mb, col0 = static_cast<size_t>(j) * nb;
        ck(cudaStreamWaitEvent(d.compute, d.in_ready[i], 0));
        ck(cudaStreamWaitEvent(d.compute, d.in_ready[8 + j], 0));
        const size_t ls_off = (row0 / q.sm) * static_cast<size_t>(q.as_rs) * ssz;
        const size_t rs_off = (col0 / q.sn) * static_cast<size_t>(q.bs_rs) * ssz;
        char* out_b = static_cast<char*>(d.out.ptr) + (row0 * q.n + col0) * esz_out;
        char* os_b = static_cast<char*>(d.os.ptr) + ((row0 / qm) * groups + (quant ? col0 / q.qn : 0)) * ssz;
        st = mxb_gemm(&sub, static_cast<char*>(d.left.ptr) + row0 * q.k, static_cast<char*>(d.right.ptr) + col0 * q.k,
                      out_b, static_cast<char*>(d.ls.ptr) + ls_off, static_cast<char*>(d.rs.ptr) + rs_off,
                      quant ? os_b : nullptr, ws_bytes ? d.ws.ptr : nullptr, ws_bytes, d.compute);
        if (st != MXB_OK) break;
        cudaEvent_t done = d.gemm_done[i * 8 + j];
        ck(cudaEventRecord(done, d.compute));
        ck(cudaStreamWaitEvent(d.d2h, done, 0));
        ck(cudaMemcpy2DAsync(static_cast<char*>(out) + (row0 * q.n + col0) * esz_out, static_cast<size_t>(q.n) * esz_out,
                          out_b, static_cast<size_t>(q.n) * esz_out, static_cast<size_t>(nb) * esz_out, mb,
                          cudaMemcpyDeviceToHost, d.d2h));
        // output scales: rows of a block are only (nb / qn) scales long, too short for efficient DMA, so they
        // go back per row block, whole rows at a time, once the row block's last column block is done
        if (quant && ++cols_done[i] == bn)
          ck(cudaMemcpyAsync(static_cast<char*>(out_scale) + (row0 / qm) * groups * ssz,
                             static_cast<char*>(d.os.ptr) + (row0 / qm) * groups * ssz,
                             static_cast<size_t>(mb / qm) * groups * ssz, cudaMemcpyDeviceToHost, d.d2h));
      }
  };
  // with out_transpose (or transposed scales) there is one block and the results are copied back whole below
  const bool whole = out_t || (quant && cs_t);
  while ((sent_a < bm || sent_b < bn) && st == MXB_OK) {
    // next operand block: keep the two operands level, `left` first
    const bool send_a = sent_a < bm && (sent_b >= bn || sent_a * bn <= sent_b * bm);
    if (send_a) {
      const size_t row0 = static_cast<size_t>(sent_a) * mb;
      ck(cudaMemcpyAsync(static_cast<char*>(d.left.ptr) + row0 * q.k, static_cast<const char*>(left) + row0 * q.k,
                      static_cast<size_t>(mb) * q.k, cudaMemcpyHostToDevice, d.h2d));
      ck(cudaEventRecord(d.in_ready[sent_a], d.h2d));
      ++sent_a;
    } else {
      const size_t col0 = static_cast<size_t>(sent_b) * nb;
      ck(cudaMemcpyAsync(static_cast<char*>(d.right.ptr) + col0 * q.k, static_cast<const char*>(right) + col0 * q.k,
                      static_cast<size_t>(nb) * q.k, cudaMemcpyHostToDevice, d.h2d));
      ck(cudaEventRecord(d.in_ready[8 + sent_b], d.h2d));
      ++sent_b;
    }
    if (!whole) launch_ready();
  }
  if (whole && st == MXB_OK) {
    ck(cudaStreamWaitEvent(d.compute, d.in_ready[0], 0));
    ck(cudaStreamWaitEvent(d.compute, d.in_ready[8], 0));
    st = mxb_gemm(&sub, d.left.ptr, d.right.ptr, d.out.ptr, d.ls.ptr, d.rs.ptr, quant ? d.os.ptr : nullptr,
                  ws_bytes ? d.ws.ptr : nullptr, ws_bytes, d.compute);
    if (st == MXB_OK) {
      ck(cudaEventRecord(d.gemm_done[0], d.compute));
      ck(cudaStreamWaitEvent(d.d2h, d.gemm_done[0], 0));
      ck(cudaMemcpyAsync(out, d.out.ptr, static_cast<size_t>(q.m) * q.n * esz_out, cudaMemcpyDeviceToHost, d.d2h));
      if (quant)
        ck(cudaMemcpyAsync(out_scale, d.os.ptr, static_cast<size_t>(q.m / qm) * groups * ssz, cudaMemcpyDeviceToHost,
                           d.d2h));
    }
  }
  cudaError_t e1 = cudaStreamSynchronize(d.h2d);
  cudaError_t e2 = cudaStreamSynchronize(d.compute);
  cudaError_t e3 = cudaStreamSynchronize(d.d2h);
  if (st != MXB_OK) return st;
  if (first_err != cudaSuccess || e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess) return MXB_ERR_CUDA;
  return MXB_OK;
}
