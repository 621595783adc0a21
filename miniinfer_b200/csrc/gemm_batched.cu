// A batch of small matrix products over strided operands, for any sizes and alignments:
//
//   out[b][m, n] = act( sum_k x[b][m, k] * w[b][n, k]  (+ bias[n]) )  (* sigmoid(row_gate[m, b]))
//
// x[b] starts at x + b * x_batch with rows lda apart, w[b] at w + b * w_batch with rows ldw apart, out[b] at
// out + b * o_batch with rows ldo apart - so the heads of a token's row (a batch stride of one head, a row stride of
// the whole row) are multiplied with a matrix per head without being repacked, and a column range of a row can be
// an operand.  Products and sums in float32, k ascending, whatever the storage type: a row's result does not depend
// on the other rows.  act: 0 none, 1 softplus (log(1 + exp(z)), z itself above 20).  row_gate: one logit per
// (row, batch) at row_gate[m * gate_stride + b]; the output rows of batch b are multiplied with its sigmoid.
//
// This is the product of the 32-bit path for strided operands, of per-head up- and down-projections of a latent
// attention, and the fallback of the bfloat16 path for inner sizes that are no multiple of 8.  Tiles of 64 x 64
// through shared memory, 16 values of k at a time, 4 x 4 outputs a thread.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

struct BatchedArgs {
  const void* x; const void* w; void* out;
  long long x_batch, w_batch, o_batch;
  int lda, ldw, ldo;
  int M, N, K;
  const float* bias;
  int act;
  const void* row_gate;
  int gate_stride;
};

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
gemm_batched_kernel(BatchedArgs a) {
  mi::grid_dependency_sync();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int b = blockIdx.z;
  const T* x = (const T*)a.x + (size_t)b * a.x_batch;
  const T* w = (const T*)a.w + (size_t)b * a.w_batch;
  TO* out = (TO*)a.out + (size_t)b * a.o_batch;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < a.K; k0 += BK) {
    for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
      const int r = idx / BK, c = idx % BK;
      const int m = m0 + r, k = k0 + c;
      xs[c][r] = (m < a.M && k < a.K) ? mi::to_float(x[(size_t)m * a.lda + k]) : 0.f;
      const int n = n0 + r;
      ws[c][r] = (n < a.N && k < a.K) ? mi::to_float(w[(size_t)n * a.ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < BK; ++c) {
      float xv[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = xs[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = ws[c][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
    float gate = 1.f;
    if (a.row_gate) gate = 1.f / (1.f + expf(-mi::to_float(((const T*)a.row_gate)[(size_t)m * a.gate_stride + b])));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      float y = acc[i][j];
      if (a.bias) y += a.bias[n];
      if (a.act == 1) y = y > 20.f ? y : log1pf(expf(y));
      out[(size_t)m * a.ldo + n] = mi::from_float<TO>(y * gate);
    }
  }
}

// Few rows (a decode step) in bfloat16: the tiled kernel would wait for global memory once per 16 values of k with one
// block a tile.  Here a warp takes one output column (batch, n): its lanes deal out k, every lane multiplies its values of
// the weight row with up to 16 rows of x, and the lanes' sums meet by shuffles.  The sum's order differs from the tiled
// kernel's, so the 32-bit path, whose results must not depend on how a request was cut, does not take this kernel.
constexpr int FEW_ROWS = 16;

template <typename TO>
__global__ void __launch_bounds__(128)
gemm_batched_few_rows_kernel(BatchedArgs a) {
  mi::grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * 4 + warp;
  const int b = blockIdx.y;
  if (n >= a.N) return;
  const __nv_bfloat16* x = (const __nv_bfloat16*)a.x + (size_t)b * a.x_batch;
  const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)b * a.w_batch + (size_t)n * a.ldw;
  float acc[FEW_ROWS];
#pragma unroll
  for (int m = 0; m < FEW_ROWS; ++m) acc[m] = 0.f;
  for (int k = lane; k < a.K; k += 32) {
    const float wv = __bfloat162float(w[k]);
#pragma unroll
    for (int m = 0; m < FEW_ROWS; ++m)
      if (m < a.M) acc[m] = fmaf(__bfloat162float(x[(size_t)m * a.lda + k]), wv, acc[m]);
  }
  TO* out = (TO*)a.out + (size_t)b * a.o_batch;
#pragma unroll
  for (int m = 0; m < FEW_ROWS; ++m) {
    if (m >= a.M) break;
    float y = mi::warp_sum(acc[m]);
    if (lane == 0) {
      if (a.bias) y += a.bias[n];
      if (a.act == 1) y = y > 20.f ? y : log1pf(expf(y));
      if (a.row_gate) y *= 1.f / (1.f + expf(-__bfloat162float(((const __nv_bfloat16*)a.row_gate)[(size_t)m * a.gate_stride + b])));
      out[(size_t)m * a.ldo + n] = mi::from_float<TO>(y);
    }
  }
}

}  // namespace

MI_API int mi_gemm_batched_few_rows(void* out, int out_dtype, const void* x, const void* w, int dtype, int batch, int M, int N, int K,
                                    int lda, long long x_batch, int ldw, long long w_batch, int ldo, long long o_batch,
                                    const float* bias, int act, const void* row_gate, int gate_stride, cudaStream_t stream) {
  MI_REQUIRE(batch > 0 && batch <= 65535 && M >= 0 && M <= FEW_ROWS && N > 0 && K > 0, "gemm_batched_few_rows: bad sizes batch=%d M=%d N=%d K=%d", batch, M, N, K);
  MI_REQUIRE(dtype == MI_BF16 && lda >= K && ldw >= K && ldo >= N && (act == 0 || act == 1), "gemm_batched_few_rows: bfloat16 operands, rows that do not overlap");
  if (M == 0) return 0;
  BatchedArgs a;
  a.x = x; a.w = w; a.out = out; a.x_batch = x_batch; a.w_batch = w_batch; a.o_batch = o_batch;
  a.lda = lda; a.ldw = ldw; a.ldo = ldo; a.M = M; a.N = N; a.K = K; a.bias = bias; a.act = act;
  a.row_gate = row_gate; a.gate_stride = gate_stride;
  dim3 grid((N + 3) / 4, batch);
  if (out_dtype == MI_BF16) mi::launch(gemm_batched_few_rows_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, a);
  else if (out_dtype == MI_F32) mi::launch(gemm_batched_few_rows_kernel<float>, grid, dim3(128), 0, stream, a);
  else return mi_fail("gemm_batched_few_rows: unknown output dtype %d", out_dtype);
  MI_LAUNCH_OK("gemm_batched_few_rows");
  return 0;
}

MI_API int mi_gemm_batched(void* out, int out_dtype, const void* x, const void* w, int dtype, int batch, int M, int N, int K,
                           int lda, long long x_batch, int ldw, long long w_batch, int ldo, long long o_batch,
                           const float* bias, int act, const void* row_gate, int gate_stride, cudaStream_t stream) {
  MI_REQUIRE(batch > 0 && batch <= 65535 && M >= 0 && N > 0 && K > 0, "gemm_batched: bad sizes batch=%d M=%d N=%d K=%d", batch, M, N, K);
  MI_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm_batched: rows overlap (lda=%d ldw=%d ldo=%d)", lda, ldw, ldo);
  MI_REQUIRE(act == 0 || act == 1, "gemm_batched: unknown activation %d", act);
  if (M == 0) return 0;
  BatchedArgs a;
  a.x = x; a.w = w; a.out = out; a.x_batch = x_batch; a.w_batch = w_batch; a.o_batch = o_batch;
  a.lda = lda; a.ldw = ldw; a.ldo = ldo; a.M = M; a.N = N; a.K = K; a.bias = bias; a.act = act;
  a.row_gate = row_gate; a.gate_stride = gate_stride;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
  MI_REQUIRE(grid.y <= 65535, "gemm_batched: M=%d is too large for one launch", M);
  if (dtype == MI_F32 && out_dtype == MI_F32) mi::launch(gemm_batched_kernel<float, float>, grid, dim3(256), 0, stream, a);
  else if (dtype == MI_BF16 && out_dtype == MI_BF16) mi::launch(gemm_batched_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, stream, a);
  else if (dtype == MI_BF16 && out_dtype == MI_F32) mi::launch(gemm_batched_kernel<__nv_bfloat16, float>, grid, dim3(256), 0, stream, a);
  else return mi_fail("gemm_batched: unsupported dtypes operands=%d out=%d", dtype, out_dtype);
  MI_LAUNCH_OK("gemm_batched");
  return 0;
}
