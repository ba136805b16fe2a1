// Linear attention with a per-head decay, as a recurrence over a 32-bit state per (sequence, head):
//
//     S_t = decay_h * S_(t-1) + k_t v_t^T        (S: dim x vdim)
//     o_t = S_t^T q_t
//
// q, k, v are act(projection) with act = x * sigmoid(x), applied here in 32-bit to the step's projections.  Columns of
// S (value channels) never mix, so a block owns a group of value channels of one (sequence, head), keeps its part of
// the state in registers for all tokens of the step, and writes it back once.  Inside a block a value channel belongs
// to SPLIT adjacent lanes, each with DPT of the head's `dim` key channels; their partial outputs meet by shuffles.
// The state lives in `state[slot][head][dim][vdim]`; a sequence that starts finds zeros there.
#include "common.cuh"

namespace bt {

constexpr int LS_TOKENS = 16;  // tokens staged in shared memory at a time

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }

template <typename T, int DPT, int SPLIT>
__global__ void __launch_bounds__(256)
lightning_scan_kernel(const T* __restrict__ proj, long long row_stride, int q_off, int k_off, int v_off,
                      float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ seq_start,
                      const float* __restrict__ decay, float* __restrict__ out, long long out_row_stride, int n_heads,
                      int dim, int vdim, int cols) {
  extern __shared__ float sm[];
  float* q_s = sm;                          // [LS_TOKENS][dim]
  float* k_s = q_s + LS_TOKENS * dim;       // [LS_TOKENS][dim]
  float* v_s = k_s + LS_TOKENS * dim;       // [LS_TOKENS][cols]
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * cols;
  const int first = seq_start[seq], n_new = seq_start[seq + 1] - first;
  const int part = threadIdx.x % SPLIT, col_local = threadIdx.x / SPLIT;
  const int col = col0 + col_local;
  const bool owns = col_local < cols && col < vdim;
  const int d0 = part * DPT;
  float* s_base = state + (((long long)slots[seq] * n_heads + head) * dim) * vdim;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) s[i] = owns && d0 + i < dim ? s_base[(long long)(d0 + i) * vdim + col] : 0.f;
  const float lam = decay[head];
  for (int t0 = 0; t0 < n_new; t0 += LS_TOKENS) {
    const int nt = min(LS_TOKENS, n_new - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * dim; i += blockDim.x) {
      const int t = i / dim, d = i - t * dim;
      const T* row = proj + (long long)(first + t0 + t) * row_stride + (long long)head * dim + d;
      q_s[i] = silu(to_float(row[q_off]));
      k_s[i] = silu(to_float(row[k_off]));
    }
    for (int i = threadIdx.x; i < nt * cols; i += blockDim.x) {
      const int t = i / cols, c = i - t * cols;
      v_s[i] = col0 + c < vdim
                   ? silu(to_float(proj[(long long)(first + t0 + t) * row_stride + v_off + (long long)head * vdim + col0 + c]))
                   : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = col_local < cols ? v_s[t * cols + col_local] : 0.f;
      const float* kt = k_s + t * dim + d0;
      const float* qt = q_s + t * dim + d0;
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        if (d0 + i < dim) {
          s[i] = fmaf(lam, s[i], kt[i] * v);
          o = fmaf(s[i], qt[i], o);
        }
      }
#pragma unroll
      for (int x = 1; x < SPLIT; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
      if (owns && part == 0) out[(long long)(first + t0 + t) * out_row_stride + (long long)head * vdim + col] = o;
    }
  }
  if (owns) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < dim) s_base[(long long)(d0 + i) * vdim + col] = s[i];
  }
}

template <typename T>
static int launch_lightning(const T* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                            const int* slots, const int* seq_start, const float* decay, float* out,
                            long long out_row_stride, int n_seqs, int n_heads, int dim, int vdim, cudaStream_t stream) {
  // DPT key channels per lane, SPLIT lanes per value channel: SPLIT * DPT >= dim
  int dpt, split;
  if (dim <= 32) { dpt = 8; split = 4; }
  else if (dim <= 64) { dpt = 8; split = 8; }
  else if (dim <= 128) { dpt = 16; split = 8; }
  else { dpt = 32; split = 8; }
  BT_CHECK(dim <= 256, "lightning_scan: %d key channels per head; the kernel takes up to 256", dim);
  const int cols = 256 / split < vdim ? 256 / split : vdim;   // value channels per block
  const dim3 grid((vdim + cols - 1) / cols, n_heads, n_seqs), block(256);
  const size_t smem = (size_t)LS_TOKENS * (2 * dim + cols) * sizeof(float);
#define BT_LS(DPT, SPLIT)                                                                                          \
  BT_PDL_OK("lightning_scan", launch_pdl(lightning_scan_kernel<T, DPT, SPLIT>, grid, block, smem, stream, 1, proj, \
                                         row_stride, q_off, k_off, v_off, state, slots, seq_start, decay, out,     \
                                         out_row_stride, n_heads, dim, vdim, cols))
  if (dpt == 8 && split == 4) BT_LS(8, 4);
  else if (dpt == 8) BT_LS(8, 8);
  else if (dpt == 16) BT_LS(16, 8);
  else BT_LS(32, 8);
#undef BT_LS
  return 0;
}

}  // namespace bt

extern "C" int bt_lightning_scan(const void* proj, long long row_stride, int q_off, int k_off, int v_off, float* state,
                                 const int* slots, const int* seq_start, const float* decay, float* out,
                                 long long out_row_stride, int n_seqs, int n_heads, int dim, int vdim, int dtype,
                                 cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && dim > 0 && vdim > 0 && n_seqs >= 0 && n_seqs <= 65535 && n_heads <= 65535,
           "lightning_scan: bad sizes seqs=%d heads=%d dim=%d vdim=%d", n_seqs, n_heads, dim, vdim);
  if (n_seqs == 0) return 0;
  if (dtype == kF32)
    return launch_lightning<float>((const float*)proj, row_stride, q_off, k_off, v_off, state, slots, seq_start, decay,
                                   out, out_row_stride, n_seqs, n_heads, dim, vdim, stream);
  if (dtype == kBF16)
    return launch_lightning<__nv_bfloat16>((const __nv_bfloat16*)proj, row_stride, q_off, k_off, v_off, state, slots,
                                           seq_start, decay, out, out_row_stride, n_seqs, n_heads, dim, vdim, stream);
  return fail("lightning_scan: unknown dtype %d", dtype);
}
