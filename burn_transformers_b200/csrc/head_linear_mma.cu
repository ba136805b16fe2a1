// Per-head products on tensor cores (bfloat16): out[t, h, :] = a[t, h, :] @ W[h] (* sigmoid(gate[t, h, :])).
// A block takes 64 tokens x 64 output columns of one head: four warps of 16 tokens each, K in pieces of 64 that pass
// through shared memory (rows an odd number of 16-byte pieces apart, so ldmatrix meets no bank twice); W[h] is [K, N]
// with N contiguous, read as the products' second operand through ldmatrix.trans.  Sums are 32-bit.
#include "decode_mma.cuh"

namespace bt {

constexpr int HL_BM = 64, HL_BN = 64, HL_BK = 64, HL_LD = 72;

__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ a, long long a_row_stride, int a_head_stride,
                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long out_row_stride,
                       int out_head_stride, const __nv_bfloat16* __restrict__ gate, long long gate_row_stride,
                       int gate_head_stride, int n_tokens, int K, int N) {
  __shared__ __align__(16) __nv_bfloat16 a_s[HL_BM * HL_LD];
  __shared__ __align__(16) __nv_bfloat16 w_s[HL_BK * HL_LD];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, t0 = blockIdx.x * HL_BM, n0 = blockIdx.z * HL_BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* ah = a + (long long)h * a_head_stride;
  const __nv_bfloat16* wh = w + (long long)h * K * N;
  float acc[HL_BN / 8][4];
#pragma unroll
  for (int j = 0; j < HL_BN / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  const unsigned a_addr = ds_smem(a_s + (warp * 16 + (lane & 15)) * HL_LD + (lane >> 4) * 8);
  const int blk = lane >> 3;
  const unsigned w_addr = ds_smem(w_s + ((blk & 1) * 8 + (lane & 7)) * HL_LD + (blk >> 1) * 8);
  // a piece of K travels global memory -> registers -> shared memory; the next piece is asked for before this one's
  // products, so its flight is hidden behind them
  uint4 a_reg[4], w_reg[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + u * 128, r = i >> 3, c = (i & 7) * 8;
      a_reg[u] = (t0 + r < n_tokens && k0 + c < K)
                     ? *reinterpret_cast<const uint4*>(ah + (long long)(t0 + r) * a_row_stride + k0 + c) : make_uint4(0u, 0u, 0u, 0u);
      w_reg[u] = (k0 + r < K && n0 + c < N) ? *reinterpret_cast<const uint4*>(wh + (long long)(k0 + r) * N + n0 + c)
                                            : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += HL_BK) {
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = tid + u * 128, r = i >> 3, c = (i & 7) * 8;
      *reinterpret_cast<uint4*>(a_s + r * HL_LD + c) = a_reg[u];
      *reinterpret_cast<uint4*>(w_s + r * HL_LD + c) = w_reg[u];
    }
    __syncthreads();
    if (k0 + HL_BK < K) fetch(k0 + HL_BK);
#pragma unroll
    for (int ks = 0; ks < HL_BK / 16; ++ks) {
      unsigned af[4];
      ds_ldmatrix_x4(af, a_addr + ks * 32);
#pragma unroll
      for (int np = 0; np < HL_BN / 16; ++np) {
        unsigned bf[4];
        ds_ldmatrix_x4_trans(bf, w_addr + (unsigned)(ks * 16 * HL_LD * 2) + np * 32);
        ds_mma(acc[2 * np], af[0], af[1], af[2], af[3], bf[0], bf[1]);
        ds_mma(acc[2 * np + 1], af[0], af[1], af[2], af[3], bf[2], bf[3]);
      }
    }
  }
  const int g = lane >> 2, qd = lane & 3;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int t = t0 + warp * 16 + g + 8 * rr;
    if (t >= n_tokens) continue;
    __nv_bfloat16* dst = out + (long long)t * out_row_stride + (long long)h * out_head_stride;
    const __nv_bfloat16* gt = gate ? gate + (long long)t * gate_row_stride + (long long)h * gate_head_stride : nullptr;
#pragma unroll
    for (int j = 0; j < HL_BN / 8; ++j) {
      const int c = n0 + j * 8 + qd * 2;
      if (c >= N) continue;
      float v0 = acc[j][2 * rr], v1 = acc[j][2 * rr + 1];
      if (gt) {
        const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gt + c));
        v0 *= 1.f / (1.f + expf(-gv.x));
        v1 *= 1.f / (1.f + expf(-gv.y));
      }
      *reinterpret_cast<unsigned*>(dst + c) = ds_pack(v0, v1);
    }
  }
}

// Whether the operands lie so that the kernel's 16-byte loads and 4-byte stores are aligned.
bool head_linear_mma_supports(const void* a, long long a_row_stride, int a_head_stride, const void* w, const void* out,
                              long long out_row_stride, int out_head_stride, const void* gate, long long gate_row_stride,
                              int gate_head_stride, int K, int N) {
  auto at = [](const void* p, int bytes) { return ((unsigned long long)p % bytes) == 0; };
  return K % 8 == 0 && N % 8 == 0 && at(a, 16) && a_row_stride % 8 == 0 && a_head_stride % 8 == 0 && at(w, 16) &&
         at(out, 4) && out_row_stride % 2 == 0 && out_head_stride % 2 == 0 &&
         (gate == nullptr || (at(gate, 4) && gate_row_stride % 2 == 0 && gate_head_stride % 2 == 0));
}

int launch_head_linear_mma(const __nv_bfloat16* a, long long a_row_stride, int a_head_stride, const __nv_bfloat16* w,
                           __nv_bfloat16* out, long long out_row_stride, int out_head_stride, const __nv_bfloat16* gate,
                           long long gate_row_stride, int gate_head_stride, int n_tokens, int n_heads, int K, int N,
                           cudaStream_t stream) {
  BT_CHECK(n_heads <= 65535 && (N + HL_BN - 1) / HL_BN <= 65535, "head_linear: %d heads or %d columns are too many", n_heads, N);
  const dim3 grid((n_tokens + HL_BM - 1) / HL_BM, n_heads, (N + HL_BN - 1) / HL_BN), block(128);
  BT_PDL_OK("head_linear_mma", launch_pdl(head_linear_mma_kernel, grid, block, 0, stream, 1, a, a_row_stride, a_head_stride,
                                          w, out, out_row_stride, out_head_stride, gate, gate_row_stride, gate_head_stride,
                                          n_tokens, K, N));
  return 0;
}

}  // namespace bt
