// float32 validation path of the fused LoRA linear: every contraction is a strided SGEMM on CUDA
// cores with float32 FMA accumulation.  tcgen05 has no float32 MMA and a single TF32 pass cannot
// hold the 1e-4 bound against the reference's f32 CPU arithmetic, so this path exists for
// correctness, not for the roofline.
#include "lora_internal.cuh"

namespace mcb {
namespace f32path {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

// C[m,n] = alpha * sum_k A(m,k) B(k,n) + beta * C[m,n] (+ bias[n]);  A(m,k) = A[m*sam + k*sak],
// B(k,n) = B[k*sbk + n*sbn];  C row-major with leading dimension ldc.
__global__ void __launch_bounds__(256)
sgemm_strided_kernel(const float* __restrict__ A, int64_t sam, int64_t sak, const float* __restrict__ B,
                     int64_t sbk, int64_t sbn, float* __restrict__ C, int64_t ldc, int M, int N, int K,
                     float alpha, float beta, const float* __restrict__ bias) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int i = threadIdx.x; i < BM * BK; i += 256) {
      // consecutive threads walk the contiguous dimension of A
      int mm, kk;
      if (sak == 1) { kk = i % BK; mm = i / BK; } else { mm = i % BM; kk = i / BM; }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? A[gm * sam + gk * sak] : 0.0f;
    }
    for (int i = threadIdx.x; i < BN * BK; i += 256) {
      int nn, kk;
      if (sbk == 1) { kk = i % BK; nn = i / BK; } else { nn = i % BN; kk = i / BN; }
      const int gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < N && gk < K) ? B[gk * sbk + gn * sbn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = alpha * acc[i][j];
      if (beta != 0.0f) v += beta * C[gm * ldc + gn];
      if (bias != nullptr) v += bias[gn];
      C[gm * ldc + gn] = v;
    }
  }
}

__global__ void add_inplace_kernel(float* __restrict__ y, const float* __restrict__ r, int64_t n) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    y[i] += r[i];
}

int add_inplace(cudaStream_t st, float* y, const float* r, int64_t n) {
  if (r == nullptr || n <= 0) return MCB_OK;
  if (r == y) return fail(MCB_ERR_UNSUPPORTED, "f32 path: residual must not alias the output");
  int64_t g = (n + 255) / 256;
  if (g > 4096) g = 4096;
  add_inplace_kernel<<<static_cast<unsigned>(g), 256, 0, st>>>(y, r, n);
  MCB_CHECK_LAUNCH("add_inplace");
  return MCB_OK;
}

int sgemm(cudaStream_t st, const float* A, int64_t sam, int64_t sak, const float* B, int64_t sbk, int64_t sbn,
          float* C, int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, float beta, const float* bias) {
  if (M <= 0 || N <= 0) return MCB_OK;
  const int64_t gy = (M + BM - 1) / BM, gx = (N + BN - 1) / BN;
  if (gy > 65535) return fail(MCB_ERR_SHAPE, "f32 path: M=%lld exceeds 65535*64 rows", (long long)M);
  dim3 grid((unsigned)gx, (unsigned)gy);
  sgemm_strided_kernel<<<grid, 256, 0, st>>>(A, sam, sak, B, sbk, sbn, C, ldc, (int)M, (int)N, (int)K, alpha, beta,
                                             bias);
  MCB_CHECK_LAUNCH("sgemm_strided");
  return MCB_OK;
}

}  // namespace

int matmul(const float* a, const float* b, float* out, int64_t M, int64_t K, int64_t N, cudaStream_t st) {
  return sgemm(st, a, K, 1, b, N, 1, out, N, M, N, K, 1.0f, 0.0f, nullptr);
}

size_t workspace_bytes(int64_t M, int64_t K, int64_t N, int64_t r) {
  (void)K; (void)N;
  return (static_cast<size_t>(M) + static_cast<size_t>(h_pitch(M))) * static_cast<size_t>(rank_padded(r)) * sizeof(float);
}

int delta_fwd(const LoraArgs& a) {
  const int64_t rp = rank_padded(a.r);
  if (a.ws_bytes < workspace_bytes(a.M, a.K, a.N, a.r) || !a.ws)
    return fail(MCB_ERR_WORKSPACE, "lora_delta_fwd(f32): workspace too small");
  float* h = static_cast<float*>(a.ws);
  // h = x A ; out = scale * (h B)   (src/training/lora.rs:323,336,339)
  if (int rc = sgemm(a.stream, (const float*)a.x, a.K, 1, a.A, a.r, 1, h, rp, a.M, a.r, a.K, 1.0f, 0.0f, nullptr))
    return rc;
  return sgemm(a.stream, h, rp, 1, a.B, a.N, 1, (float*)a.y, a.N, a.M, a.N, a.r, a.scale, 0.0f, nullptr);
}

int linear_fwd(const LoraArgs& a) {
  const int64_t pitch = h_pitch(a.M);
  const int64_t sbk = a.w_layout == MCB_W_OUT_IN ? 1 : a.N;
  const int64_t sbn = a.w_layout == MCB_W_OUT_IN ? a.K : 1;
  if (int rc = sgemm(a.stream, (const float*)a.x, a.K, 1, (const float*)a.W, sbk, sbn, (float*)a.y, a.N, a.M, a.N,
                     a.K, 1.0f, 0.0f, (const float*)a.bias))
    return rc;
  if (int rc = add_inplace(a.stream, (float*)a.y, (const float*)a.residual, a.M * a.N)) return rc;
  if (a.r == 0) return MCB_OK;
  // hs = scale * (x A), kept transposed [rp, pitch] like the bf16 path's saved intermediate
  float* hs = static_cast<float*>(a.h_save);
  if (hs == nullptr) {
    if (a.ws_bytes < workspace_bytes(a.M, a.K, a.N, a.r) || !a.ws)
      return fail(MCB_ERR_WORKSPACE, "lora_linear_fwd(f32): workspace too small");
    hs = static_cast<float*>(a.ws);
  }
  // hs[j, m] = scale * sum_k A[k, j] x[m, k]
  if (int rc = sgemm(a.stream, a.A, 1, a.r, (const float*)a.x, 1, a.K, hs, pitch, a.r, a.M, a.K, a.scale, 0.0f, nullptr))
    return rc;
  // y[m, n] += sum_j hs[j, m] B[j, n]
  return sgemm(a.stream, hs, 1, pitch, a.B, a.N, 1, (float*)a.y, a.N, a.M, a.N, a.r, 1.0f, 1.0f, nullptr);
}

int linear_bwd(const LoraArgs& a) {
  const int64_t rp = rank_padded(a.r);
  const int64_t pitch = h_pitch(a.M);
  const float* dy = static_cast<const float*>(a.dy);
  // dy W : W(k_red = n, out = k)
  const int64_t sbk = a.w_layout == MCB_W_OUT_IN ? a.K : 1;
  const int64_t sbn = a.w_layout == MCB_W_OUT_IN ? 1 : a.N;
  if (a.dx != nullptr) {
    if (int rc = sgemm(a.stream, dy, a.N, 1, (const float*)a.W, sbk, sbn, (float*)a.dx, a.K, a.M, a.K, a.N, 1.0f, 0.0f,
                       nullptr))
      return rc;
    if (int rc = add_inplace(a.stream, (float*)a.dx, (const float*)a.residual, a.M * a.K)) return rc;
  }
  if (a.r == 0) return MCB_OK;
  if (a.ws_bytes < workspace_bytes(a.M, a.K, a.N, a.r) || !a.ws)
    return fail(MCB_ERR_WORKSPACE, "lora_linear_bwd(f32): workspace too small");
  float* dh = static_cast<float*>(a.ws);                  // scale * dy B^T   [M, rp]
  float* hs_ws = dh + a.M * rp;                           // scale * x A      [rp, pitch] when not saved
  if (int rc = sgemm(a.stream, dy, a.N, 1, a.B, 1, a.N, dh, rp, a.M, a.r, a.N, a.scale, 0.0f, nullptr)) return rc;
  if (a.dx != nullptr) {
    if (int rc = sgemm(a.stream, dh, rp, 1, a.A, 1, a.r, (float*)a.dx, a.K, a.M, a.K, a.r, 1.0f, 1.0f, nullptr))
      return rc;
  }
  if (a.dA == nullptr && a.dB == nullptr) return MCB_OK;
  const float beta = a.accumulate ? 1.0f : 0.0f;
  if (a.dA != nullptr) {
    // dA[k, j] = sum_m x[m,k] dh[m,j]
    if (int rc = sgemm(a.stream, (const float*)a.x, 1, a.K, dh, rp, 1, a.dA, a.r, a.K, a.r, a.M, 1.0f, beta, nullptr))
      return rc;
  }
  if (a.dB != nullptr) {
    const float* hs = static_cast<const float*>(a.h_save);
    if (hs == nullptr) {
      if (int rc = sgemm(a.stream, a.A, 1, a.r, (const float*)a.x, 1, a.K, hs_ws, pitch, a.r, a.M, a.K, a.scale, 0.0f,
                         nullptr))
        return rc;
      hs = hs_ws;
    }
    // dB[j, n] = sum_m hs[j,m] dy[m,n]
    if (int rc = sgemm(a.stream, hs, pitch, 1, dy, a.N, 1, a.dB, a.N, a.r, a.N, a.M, 1.0f, beta, nullptr)) return rc;
  }
  return MCB_OK;
}

}  // namespace f32path
}  // namespace mcb
