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
  // with `mixed`: a block holds all value channels of its head, and instead of o the kernel leaves
  // o / rms(o) * norm_w * sigmoid(gate) (the gate's channels at g_off of the rows of proj) in `mixed`, in proj's type
  const float* norm_w;
  float eps;
  int g_off;
  void* mixed;
  long long mixed_row_stride;
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
  float* red_s = floor_s + ML_TOKENS;         // [33] for sums over the block
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
      const float read = o / (fmaxf(fabsf(nq), floor_s[t]) + 1e-6f);
      if (p.mixed) {
        const float ss = block_sum(owns && part == 0 ? read * read : 0.f, red_s);
        if (owns && part == 0) {
          const long long row = first + t0 + t;
          const int ch = head * vdim + col;
          const float gate = to_float(proj[row * p.row_stride + p.g_off + ch]);
          const float y = read / sqrtf(ss / (float)vdim + p.eps) * p.norm_w[ch] / (1.f + expf(-gate));
          reinterpret_cast<T*>(p.mixed)[row * p.mixed_row_stride + ch] = from_float<T>(y);
        }
      } else if (owns && part == 0) {
        p.out[(long long)(first + t0 + t) * p.out_row_stride + (long long)head * vdim + col] = read;
      }
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
  if (p.mixed && p.vdim > 256 / split) {      // a whole head a block: 64 value channels, more key channels a lane
    split = 4;
    dpt = p.dim <= 64 ? 16 : 32;
  }
  p.cols = 256 / split < p.vdim ? 256 / split : p.vdim;   // value channels per block
  const dim3 grid((p.vdim + p.cols - 1) / p.cols, p.n_heads, n_seqs), block(256);
  BT_CHECK(!p.mixed || grid.x == 1, "mlstm_scan: a head of %d x %d does not fit one block, the norm cannot be fused", p.dim,
           p.vdim);
  const size_t smem = (size_t)(ML_TOKENS * (2 * p.dim + p.cols + 3) + 33) * sizeof(float);
#define BT_ML(DPT, SPLIT) \
  BT_PDL_OK("mlstm_scan", launch_pdl(mlstm_scan_kernel<T, DPT, SPLIT>, grid, block, smem, stream, 1, proj, p))
  if (dpt == 8 && split == 4) BT_ML(8, 4);
  else if (dpt == 8) BT_ML(8, 8);
  else if (dpt == 16 && split == 4) BT_ML(16, 4);
  else if (dpt == 32 && split == 4) BT_ML(32, 4);
  else if (dpt == 16) BT_ML(16, 8);
  else BT_ML(32, 8);
#undef BT_ML
  return 0;
}


// ---- long runs of new tokens: the same recurrence by chunks ------------------------------------------------------
//
// With c_t the sum of the forget gates' logs b from the chunk's first token to t, a chunk that starts from
// (S_in, n_in, m_in) has, for its tokens t and s <= t,
//
//     m_t   = max(c_t + m_in, max_s (c_t - c_s + a_s))                                 (the same m_t as token by token)
//     num_t = exp(c_t + m_in - m_t) S_in^T q_t + sum_s exp(c_t - c_s + a_s - m_t) (q_t . k_s) v_s
//     den_t = exp(c_t + m_in - m_t) n_in . q_t + sum_s exp(c_t - c_s + a_s - m_t) (q_t . k_s)
//     o_t   = num_t / (max(|den_t|, exp(-m_t)) + 1e-6)
//     S_out = exp(c_L + m_in - m_L) S_in + sum_s exp(c_L - c_s + a_s - m_L) k_s v_s^T      (L: the chunk's last token)
//
// and no exponent is above zero.  mlstm_gates_kernel forms a, c and m for every token (a warp scans the running maximum:
// the maps m -> max(m + b, a) compose); mlstm_chunk_kernel the sums over s per chunk, side by side; mlstm_prefix_kernel
// walks a sequence's chunks in order and leaves each the state it starts from; mlstm_carry_kernel adds the parts with
// S_in and n_in and divides.
constexpr int MC = 64;    // tokens per chunk
constexpr int MCP = 68;   // row length of the transposed tiles

struct MlstmChunked {
  MlstmArgs a;
  float* ga;       // [rows][heads] log input gate
  float* gc;       // [rows][heads] sum of the log forget gates since the chunk's first token
  float* gm;       // [rows][heads] running maximum
  float* den;      // [rows][heads] the chunk's own part of n . q
  float* m_start;  // [seqs][chunks][heads] maximum the chunk starts from
  float* carry;    // [seqs][chunks][heads] exp(c_L + m_in - m_L)
  float* ds;       // [seqs][chunks][heads][dim][vdim] contribution, then the state the chunk starts from
  float* dn;       // [seqs][chunks][heads][dim]
  int max_chunks, col_blocks;
};

constexpr int MG_TOKENS = 2048;   // tokens whose gates lie in shared memory at a time (a multiple of the chunk)

template <typename T>
__global__ void __launch_bounds__(256) mlstm_gates_kernel(const T* __restrict__ proj, MlstmChunked c) {
  __shared__ float a_s[MG_TOKENS], b_s[MG_TOKENS];
  const MlstmArgs& p = c.a;
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, seq = blockIdx.y, H = p.n_heads;
  const int first = p.seq_start[seq], n_new = p.seq_start[seq + 1] - first;
  const float bias_i = p.i_bias[head], bias_f = p.f_bias[head];
  const int lane = threadIdx.x & 31;
  const long long slot_head = (long long)p.slots[seq] * H + head;
  float m = p.m[slot_head], m_in = m, sum = 0.f;       // (warp 0's copies are the ones that count)
  for (int base = 0; base < n_new; base += MG_TOKENS) {
    const int count = min(MG_TOKENS, n_new - base);
    __syncthreads();
    for (int t = threadIdx.x; t < count; t += blockDim.x) {
      const T* row = proj + (long long)(first + base + t) * p.row_stride + head;
      const float a = p.cap * tanhf((to_float(row[p.i_off]) + bias_i) / p.cap);
      a_s[t] = a;
      b_s[t] = log_sigmoid(p.cap * tanhf((to_float(row[p.f_off]) + bias_f) / p.cap));
      c.ga[(long long)(first + base + t) * H + head] = a;
    }
    __syncthreads();
    if (threadIdx.x >= 32) continue;
    for (int t0 = 0; t0 < count; t0 += 32) {
      const int chunk = (base + t0) / MC;
      const long long at = ((long long)seq * c.max_chunks + chunk) * H + head;
      if ((base + t0) % MC == 0) {
        sum = 0.f;
        m_in = m;
        if (lane == 0) c.m_start[at] = m;
      }
      const int t = t0 + lane;
      const bool valid = t < count;
      // the map of token t is m -> max(m + B, A); lanes past the run hold the identity
      float B = valid ? b_s[t] : 0.f, A = valid ? a_s[t] : -INFINITY;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float Bp = __shfl_up_sync(0xffffffffu, B, o), Ap = __shfl_up_sync(0xffffffffu, A, o);
        if (lane >= o) {
          A = fmaxf(Ap + B, A);
          B = Bp + B;
        }
      }
      const float m_t = fmaxf(m + B, A);
      if (valid) {
        const long long g = (long long)(first + base + t) * H + head;
        c.gc[g] = sum + B;
        c.gm[g] = m_t;
      }
      const int last = min(31, count - 1 - t0);
      m = __shfl_sync(0xffffffffu, m_t, last);
      sum += __shfl_sync(0xffffffffu, B, last);
      if (lane == 0 && ((base + t0 + 32) % MC == 0 || base + t0 + 32 >= n_new)) c.carry[at] = expf(sum + m_in - m);
    }
  }
  if (threadIdx.x == 0) p.m[slot_head] = m;
}

// grid (chunks, heads * column blocks, sequences); 256 threads as a 16 x 16 grid, thread (ty, tx) owns a 4 x 4 patch of
// every product; a block owns 64 value channels.  Tiles hold their 64 tokens along the fast axis.
template <typename T>
__global__ void __launch_bounds__(256) mlstm_chunk_kernel(const T* __restrict__ proj, MlstmChunked c) {
  const MlstmArgs& p = c.a;
  const int dim = p.dim, vdim = p.vdim, H = p.n_heads;
  extern __shared__ __align__(16) float sm[];
  float* q_t = sm;                       // [dim][MCP]   q_t[d][t]
  float* k_t = q_t + dim * MCP;          // [dim][MCP]   k_t[d][s]
  float* v_s = k_t + dim * MCP;          // [MC][64]     v_s[s][j]
  float* a_t = v_s + MC * 64;            // [MC][MCP]    a_t[s][t] = exp(c_t - c_s + a_s - m_t) (q_t . k_s), zero for s > t
  float* g_a = a_t + MC * MCP;           // [MC] a_s - c_s
  float* g_c = g_a + MC;                 // [MC] c_t - m_t
  float* w_end = g_c + MC;               // [MC] exp(c_L - c_s + a_s - m_L)
  pdl_trigger();
  pdl_wait();
  const int chunk = blockIdx.x, seq = blockIdx.z;
  const int head = blockIdx.y / c.col_blocks, col_block = blockIdx.y - head * c.col_blocks, col0 = col_block * 64;
  const int first = p.seq_start[seq], n_new = p.seq_start[seq + 1] - first;
  if (chunk * MC >= n_new) return;
  const int len = min(MC, n_new - chunk * MC);
  const long long row0 = first + (long long)chunk * MC;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  if (tid < MC) {
    float ga = 0.f, gc = 0.f, gm = 0.f;
    if (tid < len) {
      const long long g = (row0 + tid) * H + head;
      ga = c.ga[g]; gc = c.gc[g]; gm = c.gm[g];
    }
    const long long gl = (row0 + len - 1) * H + head;
    g_a[tid] = ga - gc;
    g_c[tid] = gc - gm;
    w_end[tid] = tid < len ? expf(c.gc[gl] - c.gm[gl] + ga - gc) : 0.f;
  }
  for (int i = tid; i < MC * dim; i += 256) {
    const int t = i / dim, d = i - t * dim;
    float qv = 0.f, kv = 0.f;
    if (t < len) {
      const T* row = proj + (row0 + t) * p.row_stride + (long long)head * dim + d;
      qv = to_float(row[p.q_off]) * p.q_scale;
      kv = to_float(row[p.k_off]);
    }
    q_t[d * MCP + t] = qv;
    k_t[d * MCP + t] = kv;
  }
  for (int i = tid; i < MC * 64; i += 256) {
    const int t = i >> 6, cc = i & 63;
    v_s[i] = (t < len && col0 + cc < vdim)
                 ? to_float(proj[(row0 + t) * p.row_stride + p.v_off + (long long)head * vdim + col0 + cc]) : 0.f;
  }
  __syncthreads();
  // weighted scores of the chunk: tokens t = 4 ty .. and s = 4 tx ..
  {
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    if (tx <= ty) {                      // (patches above the diagonal are zeros)
      for (int d = 0; d < dim; ++d) {
        const float4 qv = *reinterpret_cast<const float4*>(q_t + d * MCP + ty * 4);
        const float4 kv = *reinterpret_cast<const float4*>(k_t + d * MCP + tx * 4);
        const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qa[i], ka[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int sx = tx * 4 + j;
      float4 o;
      float* oa = reinterpret_cast<float*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = ty * 4 + i;
        oa[i] = (sx <= t && t < len) ? acc[i][j] * expf(g_c[t] + g_a[sx]) : 0.f;
      }
      *reinterpret_cast<float4*>(a_t + sx * MCP + ty * 4) = o;
    }
  }
  __syncthreads();
  // the parts of num_t and den_t that need no earlier chunk: tokens 4 ty .., channels 4 tx ..
  {
    float acc[4][4], den[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int s_end = min(len, ty * 4 + 4);
    for (int sx = 0; sx < s_end; ++sx) {
      const float4 av = *reinterpret_cast<const float4*>(a_t + sx * MCP + ty * 4);
      const float4 vv = *reinterpret_cast<const float4*>(v_s + sx * 64 + tx * 4);
      const float aa[4] = {av.x, av.y, av.z, av.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        den[i] += aa[i];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], va[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = ty * 4 + i;
      if (t >= len) break;
      if (tx == 0 && col_block == 0) c.den[(row0 + t) * H + head] = den[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int cc = col0 + tx * 4 + j;
        if (cc < vdim) p.out[(row0 + t) * p.out_row_stride + (long long)head * vdim + cc] = acc[i][j];
      }
    }
  }
  // the chunk's contribution to the state: key channels 4 ty .. (+ 64, ...)
  const long long cell = ((long long)seq * c.max_chunks + chunk) * H + head;
  float* dst = c.ds + cell * dim * vdim;
  for (int i0 = ty * 4; i0 < dim; i0 += 64) {
    float acc[4][4], nacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int sx = 0; sx < len; ++sx) {
      const float w = w_end[sx];
      const float4 vv = *reinterpret_cast<const float4*>(v_s + sx * 64 + tx * 4);
      const float va[4] = {vv.x * w, vv.y * w, vv.z * w, vv.w * w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float kv = i0 + i < dim ? k_t[(i0 + i) * MCP + sx] : 0.f;
        nacc[i] = fmaf(kv, w, nacc[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(kv, va[j], acc[i][j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i0 + i >= dim) break;
      if (tx == 0 && col_block == 0) c.dn[cell * dim + i0 + i] = nacc[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int cc = col0 + tx * 4 + j;
        if (cc < vdim) dst[(long long)(i0 + i) * vdim + cc] = acc[i][j];
      }
    }
  }
}

// One thread per (sequence, head, element of S or of n): walks the sequence's chunks in order; leaves in the chunk's
// cell the state that chunk STARTS from, and in the state what the last chunk leaves.
__global__ void __launch_bounds__(256) mlstm_prefix_kernel(MlstmChunked c) {
  const MlstmArgs& p = c.a;
  pdl_trigger();
  pdl_wait();
  const int seq = blockIdx.z, head = blockIdx.y, H = p.n_heads, dim = p.dim, vdim = p.vdim;
  const int e = blockIdx.x * 256 + threadIdx.x;
  if (e >= dim * (vdim + 1)) return;
  const int n_new = p.seq_start[seq + 1] - p.seq_start[seq];
  const int n_chunks = (n_new + MC - 1) / MC;
  const long long slot_head = (long long)p.slots[seq] * H + head;
  const bool is_s = e < dim * vdim;
  float* st = is_s ? p.s + slot_head * dim * vdim + e : p.n + slot_head * dim + (e - dim * vdim);
  const long long base = ((long long)seq * c.max_chunks) * H + head;
  float* cell = is_s ? c.ds + base * dim * vdim + e : c.dn + base * dim + (e - dim * vdim);
  const long long stride = (long long)H * (is_s ? dim * vdim : dim);
  float s = *st;
  for (int k = 0; k < n_chunks; k += 4) {
    float kv[4], f[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      kv[u] = k + u < n_chunks ? __ldcg(cell + (k + u) * stride) : 0.f;
      f[u] = k + u < n_chunks ? c.carry[base + (long long)(k + u) * H] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (k + u < n_chunks) {
        cell[(k + u) * stride] = s;
        s = fmaf(f[u], s, kv[u]);
      }
    }
  }
  *st = s;
}

// out[t] = (out[t] + f_t S_in^T q_t) / (max(|den_t + f_t n_in . q_t|, exp(-m_t)) + 1e-6), f_t = exp(c_t + m_in - m_t);
// grid and blocks as mlstm_chunk_kernel.
template <typename T>
__global__ void __launch_bounds__(256) mlstm_carry_kernel(const T* __restrict__ proj, MlstmChunked c) {
  const MlstmArgs& p = c.a;
  const int dim = p.dim, vdim = p.vdim, H = p.n_heads;
  extern __shared__ __align__(16) float sm[];
  float* q_t = sm;                 // [dim][MCP], q_t[d][t] already times f_t
  float* s_s = q_t + dim * MCP;    // [dim][64]
  float* n_s = s_s + dim * 64;     // [dim]
  float* f_s = n_s + dim;          // [MC]
  float* div_s = f_s + MC;         // [MC] the divisor of token t
  pdl_trigger();
  pdl_wait();
  const int chunk = blockIdx.x, seq = blockIdx.z;
  const int head = blockIdx.y / c.col_blocks, col0 = (blockIdx.y - head * c.col_blocks) * 64;
  const int first = p.seq_start[seq], n_new = p.seq_start[seq + 1] - first;
  if (chunk * MC >= n_new) return;
  const int len = min(MC, n_new - chunk * MC);
  const long long row0 = first + (long long)chunk * MC;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const long long cell = ((long long)seq * c.max_chunks + chunk) * H + head;
  if (tid < MC) {
    const long long g = (row0 + tid) * H + head;
    f_s[tid] = tid < len ? expf(c.gc[g] + c.m_start[cell] - c.gm[g]) : 0.f;
  }
  for (int d = tid; d < dim; d += 256) n_s[d] = c.dn[cell * dim + d];
  __syncthreads();
  for (int i = tid; i < MC * dim; i += 256) {
    const int t = i / dim, d = i - t * dim;
    q_t[d * MCP + t] = t < len ? to_float(proj[(row0 + t) * p.row_stride + p.q_off + (long long)head * dim + d]) *
                                     p.q_scale * f_s[t] : 0.f;
  }
  const float* src = c.ds + cell * dim * vdim + col0;
  for (int i = tid; i < dim * 64; i += 256) {
    const int d = i >> 6, cc = i & 63;
    s_s[i] = col0 + cc < vdim ? src[(long long)d * vdim + cc] : 0.f;
  }
  __syncthreads();
  if (tid < len) {
    float nq = 0.f;
    for (int d = 0; d < dim; ++d) nq = fmaf(q_t[d * MCP + tid], n_s[d], nq);
    const long long g = (row0 + tid) * H + head;
    div_s[tid] = fmaxf(fabsf(c.den[g] + nq), expf(-c.gm[g])) + 1e-6f;
  }
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int d = 0; d < dim; ++d) {
    const float4 qv = *reinterpret_cast<const float4*>(q_t + d * MCP + ty * 4);
    const float4 sv = *reinterpret_cast<const float4*>(s_s + d * 64 + tx * 4);
    const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, sa[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qa[i], sa[j], acc[i][j]);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = ty * 4 + i;
    if (t >= len) break;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int cc = col0 + tx * 4 + j;
      if (cc < vdim) {
        float* o = p.out + (row0 + t) * p.out_row_stride + (long long)head * vdim + cc;
        *o = (*o + acc[i][j]) / div_s[t];
      }
    }
  }
}

static long long mlstm_scratch_floats(long long n_rows, int n_seqs, int max_new, int n_heads, int dim, int vdim) {
  const long long chunks = (max_new + MC - 1) / MC;
  const long long cells = (long long)n_seqs * chunks * n_heads;
  return 4 * (n_rows * n_heads + 4) + 2 * (cells + 4) + cells * dim * (vdim + 1) + 64;
}

template <typename T>
static int launch_mlstm_chunked(const T* proj, MlstmArgs p, float* scratch, long long n_rows, int max_new, int n_seqs,
                                cudaStream_t stream) {
  MlstmChunked c;
  c.a = p;
  c.max_chunks = (max_new + MC - 1) / MC;
  c.col_blocks = (p.vdim + 63) / 64;
  const long long per_row = (n_rows * p.n_heads + 3) / 4 * 4;
  const long long cells = (long long)n_seqs * c.max_chunks * p.n_heads, cells4 = (cells + 3) / 4 * 4;
  c.ga = scratch;
  c.gc = c.ga + per_row;
  c.gm = c.gc + per_row;
  c.den = c.gm + per_row;
  c.m_start = c.den + per_row;
  c.carry = c.m_start + cells4;
  c.ds = c.carry + cells4;
  c.dn = c.ds + cells * p.dim * p.vdim;
  BT_CHECK((long long)p.n_heads * c.col_blocks <= 65535, "mlstm_scan: %d heads x %d column blocks are too many", p.n_heads,
           c.col_blocks);
  const dim3 grid(c.max_chunks, p.n_heads * c.col_blocks, n_seqs), block(256);
  const size_t smem_a = ((size_t)2 * p.dim * MCP + (size_t)MC * 64 + (size_t)MC * MCP + 3 * MC) * sizeof(float);
  const size_t smem_c = ((size_t)p.dim * MCP + (size_t)p.dim * 64 + p.dim + 2 * MC) * sizeof(float);
  auto chunk_kernel = mlstm_chunk_kernel<T>;
  auto carry_kernel = mlstm_carry_kernel<T>;
  if (smem_a > 48 * 1024)
    BT_CHECK(cudaFuncSetAttribute(chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a) == cudaSuccess,
             "mlstm_scan: cannot reserve %zu bytes of shared memory", smem_a);
  if (smem_c > 48 * 1024)
    BT_CHECK(cudaFuncSetAttribute(carry_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c) == cudaSuccess,
             "mlstm_scan: cannot reserve %zu bytes of shared memory", smem_c);
  BT_PDL_OK("mlstm_gates", launch_pdl(mlstm_gates_kernel<T>, dim3(p.n_heads, n_seqs), block, 0, stream, 1, proj, c));
  BT_PDL_OK("mlstm_chunk", launch_pdl(chunk_kernel, grid, block, smem_a, stream, 1, proj, c));
  BT_PDL_OK("mlstm_prefix", launch_pdl(mlstm_prefix_kernel, dim3((p.dim * (p.vdim + 1) + 255) / 256, p.n_heads, n_seqs),
                                       block, 0, stream, 1, c));
  BT_PDL_OK("mlstm_carry", launch_pdl(carry_kernel, grid, block, smem_c, stream, 1, proj, c));
  return 0;
}

}  // namespace bt

// Whether bt_mlstm_scan can hold a whole head in one block, and so apply the per-head norm and the gate itself.
extern "C" int bt_mlstm_scan_fuses(int dim, int vdim) { return vdim <= 32 || (vdim <= 64 && dim <= 128); }

// norm_w .. mixed_row_stride: null / 0, or (where bt_mlstm_scan_fuses) the per-head RMS norm's weight [heads * vdim], its
// eps, the channel of the output gate in the rows of proj, and where the normed and gated rows go (proj's type); `out`
// is then not written.
extern "C" int bt_mlstm_scan(const void* proj, long long row_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                             const float* i_bias, const float* f_bias, float cap, float q_scale, float* s, float* n,
                             float* m, const int* slots, const int* seq_start, float* out, long long out_row_stride,
                             const float* norm_w, float eps, int g_off, void* mixed, long long mixed_row_stride,
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
  BT_CHECK(mixed == nullptr || (norm_w != nullptr && bt_mlstm_scan_fuses(dim, vdim)),
           "mlstm_scan: the norm of heads of %d x %d cannot be fused", dim, vdim);
  p.norm_w = norm_w; p.eps = eps; p.g_off = g_off; p.mixed = mixed; p.mixed_row_stride = mixed_row_stride;
  if (dtype == kF32) return launch_mlstm<float>((const float*)proj, p, n_seqs, stream);
  if (dtype == kBF16) return launch_mlstm<__nv_bfloat16>((const __nv_bfloat16*)proj, p, n_seqs, stream);
  return fail("mlstm_scan: unknown dtype %d", dtype);
}

// Floats of scratch the chunked form needs for a step of `n_rows` tokens whose longest run has `max_new`.
extern "C" long long bt_mlstm_chunked_scratch_floats(long long n_rows, int n_seqs, int max_new, int n_heads, int dim,
                                                     int vdim) {
  return bt::mlstm_scratch_floats(n_rows, n_seqs, max_new, n_heads, dim, vdim);
}

// The recurrence for steps that bring long runs of tokens: the same results as bt_mlstm_scan (beyond rounding), the
// chunks of a run worked side by side.  `max_new`: no sequence of the step brings more tokens than this; `n_rows`: the
// step's tokens.
extern "C" int bt_mlstm_chunked(const void* proj, long long row_stride, int q_off, int k_off, int v_off, int i_off,
                                int f_off, const float* i_bias, const float* f_bias, float cap, float q_scale, float* s,
                                float* n, float* m, const int* slots, const int* seq_start, float* out,
                                long long out_row_stride, float* scratch, long long n_rows, int max_new, int n_seqs,
                                int n_heads, int dim, int vdim, int dtype, cudaStream_t stream) {
  using namespace bt;
  BT_CHECK(n_heads > 0 && dim > 0 && dim <= 256 && vdim > 0 && n_seqs >= 0 && n_seqs <= 65535 && n_heads <= 65535 &&
               max_new > 0 && n_rows >= 0 && scratch,
           "mlstm_chunked: bad sizes seqs=%d heads=%d dim=%d vdim=%d max_new=%d", n_seqs, n_heads, dim, vdim, max_new);
  BT_CHECK(cap > 0.f, "mlstm_chunked: the gates' cap must be positive");
  if (n_seqs == 0) return 0;
  MlstmArgs p;
  p.row_stride = row_stride;
  p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.i_off = i_off; p.f_off = f_off;
  p.i_bias = i_bias; p.f_bias = f_bias; p.cap = cap; p.q_scale = q_scale;
  p.s = s; p.n = n; p.m = m; p.slots = slots; p.seq_start = seq_start; p.out = out; p.out_row_stride = out_row_stride;
  p.n_heads = n_heads; p.dim = dim; p.vdim = vdim; p.cols = 64;
  p.norm_w = nullptr; p.eps = 0.f; p.g_off = 0; p.mixed = nullptr; p.mixed_row_stride = 0;
  if (dtype == kF32) return launch_mlstm_chunked<float>((const float*)proj, p, scratch, n_rows, max_new, n_seqs, stream);
  if (dtype == kBF16)
    return launch_mlstm_chunked<__nv_bfloat16>((const __nv_bfloat16*)proj, p, scratch, n_rows, max_new, n_seqs, stream);
  return fail("mlstm_chunked: unknown dtype %d", dtype);
}
