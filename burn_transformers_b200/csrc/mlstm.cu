// A matrix memory with exponential gates, as a recurrence over a 32-bit state per (sequence, head):
//
//     a_t = cap tanh((x_i,t + bias_i) / cap)                      log of the input gate
//     b_t = log sigmoid(cap tanh((x_f,t + bias_f) / cap))         log of the forget gate
//     m_t = max(b_t + m_(t-1), a_t)                               running maximum (0 before the first token)
//     S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T       (S: dim x vdim)
//     n_t = the same with k_t alone                                            (n: dim)
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// x_i, x_f, q, k, v are columns of the step's projections; q is scaled here (dim^-1/2 is handed in).  Everything
// from the gates on is 32-bit.  Columns of S (value channels) never mix, so a block owns a group of value channels of
// one (sequence, head) and keeps its part of S in registers for all tokens of the step; n and m are small and every
// block keeps its own copy (the block of the first channel group writes them back).  A value channel belongs to SPLIT
// adjacent lanes, each with DPT of the head's key channels; partial sums meet by shuffles.
// State: s[slot][head][dim][vdim], n[slot][head][dim], m[slot][head]; a sequence that starts finds zeros there.
#include "common.cuh"

namespace bt {

constexpr int ML_TOKENS = 16;  // tokens staged in shared memory at a time

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

struct MlstmArgs {
  long long row_stride;
  int q_off, k_off, v_off, i_off, f_off;
  const float* i_bias;
  const float* f_bias;
  float cap, q_scale;
  float* s;
  float* n;
  float* m;
  const int* slots;
  const int* seq_start;
  float* out;
  long long out_row_stride;
  int n_heads, dim, vdim, cols;
};

template <typename T, int DPT, int SPLIT>
__global__ void __launch_bounds__(256) mlstm_scan_kernel(const T* __restrict__ proj, MlstmArgs p) {
  extern __shared__ float sm[];
  const int dim = p.dim, vdim = p.vdim, cols = p.cols;
  float* q_s = sm;                            // [ML_TOKENS][dim]
  float* k_s = q_s + ML_TOKENS * dim;         // [ML_TOKENS][dim]
  float* v_s = k_s + ML_TOKENS * dim;         // [ML_TOKENS][cols]
  float* keep_s = v_s + ML_TOKENS * cols;     // [ML_TOKENS] exp(b + m_old - m_new)
  float* take_s = keep_s + ML_TOKENS;         // [ML_TOKENS] exp(a - m_new)
  float* floor_s = take_s + ML_TOKENS;        // [ML_TOKENS] exp(-m_new)
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * cols;
  const int first = p.seq_start[seq], n_new = p.seq_start[seq + 1] - first;
  const int part = threadIdx.x % SPLIT, col_local = threadIdx.x / SPLIT;
  const int col = col0 + col_local;
  const bool owns = col_local < cols && col < vdim;
  const int d0 = part * DPT;
  const long long slot_head = (long long)p.slots[seq] * p.n_heads + head;
  float* s_base = p.s + slot_head * dim * vdim;
  float* n_base = p.n + slot_head * dim;
  float s[DPT], nn[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    s[i] = owns && d0 + i < dim ? s_base[(long long)(d0 + i) * vdim + col] : 0.f;
    nn[i] = d0 + i < dim ? n_base[d0 + i] : 0.f;
  }
  float m = p.m[slot_head];                   // (only thread 0's copy is advanced)
  const float bias_i = p.i_bias[head], bias_f = p.f_bias[head];
  for (int t0 = 0; t0 < n_new; t0 += ML_TOKENS) {
    const int nt = min(ML_TOKENS, n_new - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * dim; i += blockDim.x) {
      const int t = i / dim, d = i - t * dim;
      const T* row = proj + (long long)(first + t0 + t) * p.row_stride + (long long)head * dim + d;
      q_s[i] = to_float(row[p.q_off]) * p.q_scale;
      k_s[i] = to_float(row[p.k_off]);
    }
    for (int i = threadIdx.x; i < nt * cols; i += blockDim.x) {
      const int t = i / cols, c = i - t * cols;
      v_s[i] = col0 + c < vdim
                   ? to_float(proj[(long long)(first + t0 + t) * p.row_stride + p.v_off + (long long)head * vdim + col0 + c])
                   : 0.f;
    }
    // the gates' nonlinearities side by side, then the running maximum token after token
    if (threadIdx.x < nt) {
      const T* row = proj + (long long)(first + t0 + threadIdx.x) * p.row_stride + head;
      keep_s[threadIdx.x] = log_sigmoid(p.cap * tanhf((to_float(row[p.f_off]) + bias_f) / p.cap));
      take_s[threadIdx.x] = p.cap * tanhf((to_float(row[p.i_off]) + bias_i) / p.cap);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int t = 0; t < nt; ++t) {
        const float b = keep_s[t], a = take_s[t];
        const float m_new = fmaxf(b + m, a);
        keep_s[t] = expf(b + m - m_new);
        take_s[t] = expf(a - m_new);
        floor_s[t] = expf(-m_new);
        m = m_new;
      }
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float v = col_local < cols ? v_s[t * cols + col_local] : 0.f;
      const float keep = keep_s[t], take = take_s[t];
      const float* kt = k_s + t * dim + d0;
      const float* qt = q_s + t * dim + d0;
      float o = 0.f, nq = 0.f;
#pragma unroll
      for (int i = 0; i < DPT; ++i) {
        if (d0 + i < dim) {
          const float tk = take * kt[i];
          s[i] = fmaf(keep, s[i], tk * v);
          nn[i] = fmaf(keep, nn[i], tk);
          o = fmaf(s[i], qt[i], o);
          nq = fmaf(nn[i], qt[i], nq);
        }
      }
#pragma unroll
      for (int x = 1; x < SPLIT; x <<= 1) {
        o += __shfl_xor_sync(0xffffffffu, o, x);
        nq += __shfl_xor_sync(0xffffffffu, nq, x);
      }
      if (owns && part == 0)
        p.out[(long long)(first + t0 + t) * p.out_row_stride + (long long)head * vdim + col] =
            o / (fmaxf(fabsf(nq), floor_s[t]) + 1e-6f);
    }
  }
  if (owns) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < dim) s_base[(long long)(d0 + i) * vdim + col] = s[i];
  }
  if (blockIdx.x == 0 && col_local == 0) {
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (d0 + i < dim) n_base[d0 + i] = nn[i];
    if (threadIdx.x == 0) p.m[slot_head] = m;
  }
}

template <typename T>
static int launch_mlstm(const T* proj, MlstmArgs p, int n_seqs, cudaStream_t stream) {
  // DPT key channels per lane, SPLIT lanes per value channel: SPLIT * DPT >= dim
  int dpt, split;
  if (p.dim <= 32) { dpt = 8; split = 4; }
  else if (p.dim <= 64) { dpt = 8; split = 8; }
  else if (p.dim <= 128) { dpt = 16; split = 8; }
  else { dpt = 32; split = 8; }
  p.cols = 256 / split < p.vdim ? 256 / split : p.vdim;   // value channels per block
  const dim3 grid((p.vdim + p.cols - 1) / p.cols, p.n_heads, n_seqs), block(256);
  const size_t smem = (size_t)ML_TOKENS * (2 * p.dim + p.cols + 3) * sizeof(float);
#define BT_ML(DPT, SPLIT) \
  BT_PDL_OK("mlstm_scan", launch_pdl(mlstm_scan_kernel<T, DPT, SPLIT>, grid, block, smem, stream, 1, proj, p))
  if (dpt == 8 && split == 4) BT_ML(8, 4);
  else if (dpt == 8) BT_ML(8, 8);
  else if (dpt == 16) BT_ML(16, 8);
  else BT_ML(32, 8);
#undef BT_ML
  return 0;
}

}  // namespace bt

extern "C" int bt_mlstm_scan(const void* proj, long long row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                             const float* i_bias, const float* f_bias, float cap, float q_scale, float* s, float* n,
                             float* m, const int* slots, const int* seq_start, float* out, long long out_row_stride,
                             int n_seqs, int n_heads, int dim, int vdim, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && dim > 0 && dim <= 256 && vdim > 0 && n_seqs >= 0 && n_seqs <= 65535 && n_heads <= 65535,
           "mlstm_scan: bad sizes seqs=%d heads=%d dim=%d vdim=%d (up to 256 key channels a head)", n_seqs, n_heads, dim,
           vdim);
  BT_CHECK(cap > 0.f, "mlstm_scan: the gates' cap must be positive");
  if (n_seqs == 0) return 0;
  MlstmArgs p;
  p.row_stride = row_stride;
  p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.i_off = i_off; p.f_off = f_off;
  p.i_bias = i_bias; p.f_bias = f_bias; p.cap = cap; p.q_scale = q_scale;
  p.s = s; p.n = n; p.m = m; p.slots = slots; p.seq_start = seq_start; p.out = out; p.out_row_stride = out_row_stride;
  p.n_heads = n_heads; p.dim = dim; p.vdim = vdim; p.cols = 0;
  if (dtype == kF32) return launch_mlstm<float>((const float*)proj, p, n_seqs, stream);
  if (dtype == kBF16) return launch_mlstm<__nv_bfloat16>((const __nv_bfloat16*)proj, p, n_seqs, stream);
  return fail("mlstm_scan: unknown dtype %d", dtype);
}
