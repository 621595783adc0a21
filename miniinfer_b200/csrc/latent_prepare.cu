// Attention through a latent: what stands between the down-projections and the attention kernels.
//
// Of a token only a latent c (C values, RMS-normed with a weight) and one rotated key part shared by all heads (R
// values) are kept.  Per head the unrotated key is W_uk c and the value W_uv c, so a head's score is
//   (W_uk^T q_plain) . c + q_rot . k_rot
// and its output W_uv (sum_j p_j c_j): the keys' and values' up-projections move to the query and to the output, and
// attention runs over one shared key/value head whose key row is [c | k_rot] and whose value row is c.
//
//   latent_down:  from the fused down-projection rows - the query latent (Q values at q_off) and the key/value row
//                 (C + R values at kv_off) - the normed query latent into a buffer of its own, the normed c and the
//                 rotated k_rot into the layer's pages (key row [c | k_rot | 0], value row [c | 0]);
//   latent_query: the rotated part of every query head, rotated, into its place behind the C values that the product
//                 with W_uk fills, in the packed query rows [token, head, cache head size].
//
// Norms, angles and rotations in float32; a table row holds cos of R / 2 angles, then their sines; value i pairs
// with value i + R / 2 (halves) or 2i with 2i + 1 (interleaved): (u, v) -> (u cos - v sin, v cos + u sin).
#include "common.cuh"

namespace {

__device__ __forceinline__ float rotated(const float* x, int d, int R, int interleaved, const float* cs) {
  const int half = R / 2;
  const bool first = interleaved ? !(d & 1) : d < half;
  const int pi = interleaved ? d >> 1 : (first ? d : d - half);
  const int partner = interleaved ? d ^ 1 : (first ? d + half : d - half);
  const float c = cs[pi], s = cs[half + pi];
  return first ? x[d] * c - x[partner] * s : x[d] * c + x[partner] * s;
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_down_kernel(const T* __restrict__ down, int ld, int q_off, int kv_off, int Q, int C, int R, int hdp,
                   const float* __restrict__ q_w, const float* __restrict__ kv_w, float eps, T* __restrict__ cq_out,
                   const float* __restrict__ rope, const int* __restrict__ positions, int interleaved,
                   const int* __restrict__ slot_mapping, T* __restrict__ kv_layer, int page_size) {
  __shared__ float scratch[33];
  extern __shared__ float kr[];                  // the R unrotated values of the shared key part
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  mi::grid_dependency_sync();
  const T* row = down + (size_t)t * ld;
  if (cq_out) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < Q; i += blockDim.x) {
      const float v = mi::to_float(row[q_off + i]);
      ss += v * v;
    }
    const float rstd = 1.f / sqrtf(mi::block_sum(ss, scratch) / (float)Q + eps);
    for (int i = threadIdx.x; i < Q; i += blockDim.x)
      cq_out[(size_t)t * Q + i] = mi::from_float<T>(q_w[i] * (mi::to_float(row[q_off + i]) * rstd));
  }
  if (slot < 0) return;
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const float v = mi::to_float(row[kv_off + i]);
    ss += v * v;
  }
  for (int i = threadIdx.x; i < R; i += blockDim.x) kr[i] = mi::to_float(row[kv_off + C + i]);
  const float rstd = 1.f / sqrtf(mi::block_sum(ss, scratch) / (float)C + eps);     // its barriers also publish kr
  const int page = slot / page_size, off = slot % page_size;
  T* krow = kv_layer + (((size_t)page * 2 + 0) * page_size + off) * hdp;
  T* vrow = kv_layer + (((size_t)page * 2 + 1) * page_size + off) * hdp;
  const float* cs = rope + (size_t)pos * R;
  for (int i = threadIdx.x; i < hdp; i += blockDim.x) {
    float kval = 0.f, vval = 0.f;
    if (i < C) kval = vval = kv_w[i] * (mi::to_float(row[kv_off + i]) * rstd);
    else if (i < C + R) kval = rotated(kr, i - C, R, interleaved, cs);
    krow[i] = mi::from_float<T>(kval);
    vrow[i] = mi::from_float<T>(vval);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_query_kernel(const T* __restrict__ q, int ldq, int H, int D, int R, int C, int hdp, T* __restrict__ q_out,
                    const float* __restrict__ rope, const int* __restrict__ positions, int interleaved) {
  extern __shared__ float qr[];                  // [warps][R]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int pos = positions[t];
  mi::grid_dependency_sync();
  const float* cs = rope + (size_t)pos * R;
  float* x = qr + (size_t)warp * R;
  for (int h = blockIdx.y * warps + warp; h < H; h += warps * gridDim.y) {
    const T* src = q + (size_t)t * ldq + (size_t)h * (D + R) + D;
    for (int i = lane; i < R; i += 32) x[i] = mi::to_float(src[i]);
    __syncwarp();
    T* dst = q_out + ((size_t)t * H + h) * hdp + C;
    for (int i = lane; i < hdp - C; i += 32) dst[i] = mi::from_float<T>(i < R ? rotated(x, i, R, interleaved, cs) : 0.f);
    __syncwarp();
  }
}

}  // namespace

MI_API int mi_latent_down(const void* down, int dtype, int ld, int q_off, int kv_off, int T, int Q, int C, int R, int hdp,
                          const float* q_w, const float* kv_w, float eps, void* cq_out, const float* rope, const int* positions,
                          int interleaved, const int* slot_mapping, void* kv_layer, int page_size, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && Q > 0 && C > 0 && R > 0 && R % 2 == 0 && hdp >= C + R, "latent_down: bad sizes Q=%d C=%d R=%d cache head size %d", Q, C, R, hdp);
  MI_REQUIRE(rope != nullptr && positions != nullptr && eps > 0.f, "latent_down: the rotation table, positions and eps are needed");
  MI_REQUIRE(slot_mapping == nullptr || (kv_layer != nullptr && page_size > 0), "latent_down: a store needs the cache layer");
  MI_REQUIRE(R * sizeof(float) <= 32 * 1024, "latent_down: rotated part of %d values is too long", R);
  if (T == 0) return 0;
  const size_t smem = (size_t)R * sizeof(float);
  if (dtype == MI_BF16)
    mi::launch(latent_down_kernel<__nv_bfloat16>, dim3(T), dim3(128), smem, stream, (const __nv_bfloat16*)down, ld, q_off, kv_off, Q, C, R, hdp,
               q_w, kv_w, eps, (__nv_bfloat16*)cq_out, rope, positions, interleaved, slot_mapping, (__nv_bfloat16*)kv_layer, page_size);
  else if (dtype == MI_F32)
    mi::launch(latent_down_kernel<float>, dim3(T), dim3(128), smem, stream, (const float*)down, ld, q_off, kv_off, Q, C, R, hdp,
               q_w, kv_w, eps, (float*)cq_out, rope, positions, interleaved, slot_mapping, (float*)kv_layer, page_size);
  else return mi_fail("latent_down: unknown dtype %d", dtype);
  MI_LAUNCH_OK("latent_down");
  return 0;
}

MI_API int mi_latent_query(const void* q, int dtype, int ldq, int T, int H, int D, int R, int C, int hdp, void* q_out,
                           const float* rope, const int* positions, int interleaved, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && H > 0 && D > 0 && R > 0 && R % 2 == 0 && hdp >= C + R, "latent_query: bad sizes");
  MI_REQUIRE(R * 4 * sizeof(float) <= 32 * 1024, "latent_query: rotated part of %d values is too long", R);
  if (T == 0) return 0;
  const size_t smem = (size_t)4 * R * sizeof(float);
  dim3 grid(T, (H + 3) / 4);
  if (dtype == MI_BF16)
    mi::launch(latent_query_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)q, ldq, H, D, R, C, hdp,
               (__nv_bfloat16*)q_out, rope, positions, interleaved);
  else if (dtype == MI_F32)
    mi::launch(latent_query_kernel<float>, grid, dim3(128), smem, stream, (const float*)q, ldq, H, D, R, C, hdp, (float*)q_out,
               rope, positions, interleaved);
  else return mi_fail("latent_query: unknown dtype %d", dtype);
  MI_LAUNCH_OK("latent_query");
  return 0;
}
