// Mixers that carry a state from token to token instead of reading a cache of keys: the short causal convolution
// in front of them, the selective scan (a diagonal state-space recurrence whose step size, input and output maps
// depend on the token) and the gated delta rule (a matrix state per head that decays per key channel and is
// corrected towards the new value along the new key).
//
// A step brings, for each of its items, q_len[b] new tokens in rows q_start[b] .. of the activations; the item's
// state lives in row seq_slot[b] of the layer's state tensor, float32, zero when the request was admitted.  A kernel
// walks an item's tokens in order, starting from the stored state and leaving the state after the last token, so the
// result at a position does not depend on how the request was cut into steps or on what else is in the batch.  All
// arithmetic of the recurrences - decays, their logarithms, softplus, exponentials, step sizes, gates, unit norms,
// the state and the sums over it - is float32; activations are read and written in the storage type.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// ------------------------------------------------------------------------------------------------------------
// Short causal convolution over time, per channel: out[t, c] = act(bias[c] + sum_k w[c, taps - 1 - k] * in[t - k, c]),
// the inputs before the step's first token coming from the item's state (the last taps - 1 inputs of the request,
// oldest first, zeros before its start).  A thread per (token, channel).
constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(T* __restrict__ out, int ldo, const T* __restrict__ x, int ldx, const float* __restrict__ w,
                   const float* __restrict__ bias, const float* __restrict__ state, long long state_stride,
                   const int* __restrict__ token_item, const int* __restrict__ q_start, const int* __restrict__ seq_slot,
                   int C, int taps, int silu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t = blockIdx.y;
  const int item = token_item[t];
  const int j = t - q_start[item];                         // index of the token among the item's new tokens
  const int slot = seq_slot[item];
  mi::grid_dependency_sync();
  if (c >= C) return;
  const float* st = state + (size_t)slot * state_stride;   // [taps - 1][C]
  float acc = bias ? bias[c] : 0.f;
  for (int k = taps - 1; k >= 0; --k) {                    // oldest input first
    const int jj = j - k;
    const float v = jj >= 0 ? mi::to_float(x[(size_t)(t - k) * ldx + c]) : st[(size_t)(taps - 1 + jj) * C + c];
    acc = fmaf(w[(size_t)c * taps + (taps - 1 - k)], v, acc);
  }
  if (silu) acc = silu_f(acc);
  out[(size_t)t * ldo + c] = mi::from_float<T>(acc);
}

// After the convolution has run: the state becomes the last taps - 1 inputs of the request.  A thread per (item, channel).
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_kernel(float* __restrict__ state, long long state_stride, const T* __restrict__ x, int ldx,
                  const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ seq_slot,
                  int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int item = blockIdx.y;
  const int row0 = q_start[item], n = q_len[item], slot = seq_slot[item];
  mi::grid_dependency_sync();
  if (c >= C) return;
  float* st = state + (size_t)slot * state_stride;
  float keep[MAX_TAPS];
  const int S = taps - 1;
#pragma unroll
  for (int r = 0; r < MAX_TAPS; ++r) {
    if (r >= S) break;
    const int jj = n - S + r;                               // index among the new tokens; negative: an older input
    keep[r] = jj >= 0 ? mi::to_float(x[(size_t)(row0 + jj) * ldx + c]) : st[(size_t)(S + jj) * C + c];
  }
#pragma unroll
  for (int r = 0; r < MAX_TAPS; ++r) {
    if (r >= S) break;
    st[(size_t)r * C + c] = keep[r];
  }
}

// ------------------------------------------------------------------------------------------------------------
// Selective scan.  Per channel c and state index n, token after token:
//   dt = softplus(dt_in[t, c] + dt_bias[c]);  S[c, n] <- exp(dt * A[c, n]) * S[c, n] + dt * u[t, c] * B[t, n]
//   y[t, c] = (sum_n S[c, n] * C[t, n] + D[c] * u[t, c]) * silu(z[t, c]),      A = -exp(A_log)
// A channel's states are dealt to P neighbouring lanes, SPT to each; their partial sums meet by shuffles.
constexpr int SPT = 8;
constexpr int SCAN_CHUNK = 16;    // tokens whose inputs are fetched together
constexpr int SCAN_THREADS = 64;

template <typename T>
struct ScanArgs {
  T* y; int ldy;
  const T* u; int ldu;          // the convolved, activated input
  const T* dt_in; int lddt;     // the step-size projection, before bias and softplus
  const T* bc; int ldbc;        // B at column b_off, C at column c_off of the same rows
  int b_off, c_off;
  const T* z; int ldz;          // the gate's input
  const float* dt_bias; const float* A_log; const float* D;
  float* state; long long state_stride;   // [slot][inner][N]
  const int* q_start; const int* q_len; const int* seq_slot;
  int inner, N, P;
};

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(ScanArgs<T> a) {
  const int item = blockIdx.y;
  const int per_block = SCAN_THREADS / a.P;
  const int c = blockIdx.x * per_block + threadIdx.x / a.P;
  const int part = threadIdx.x % a.P;
  const int row0 = a.q_start[item], n_new = a.q_len[item], slot = a.seq_slot[item];
  const bool live = c < a.inner;
  const int cc = live ? c : 0;
  float A[SPT];
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    const int n = part * SPT + i;
    A[i] = n < a.N ? -expf(a.A_log[(size_t)cc * a.N + n]) : 0.f;
  }
  const float dtb = a.dt_bias[cc], Dc = a.D[cc];
  mi::grid_dependency_sync();
  float* st = a.state + (size_t)slot * a.state_stride + (size_t)cc * a.N;
  float S[SPT];
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    const int n = part * SPT + i;
    S[i] = (live && n < a.N) ? st[n] : 0.f;
  }
  // The tokens go by in chunks: a chunk's B and C rows into shared memory and its step sizes, inputs and gates into
  // registers, all loads issued together, and only then the recurrence over the chunk - so the latency of the loads is
  // paid once a chunk and not once a token.
  extern __shared__ float bc_s[];               // [SCAN_CHUNK][2][N]
  const int N = a.N;
  for (int c0 = 0; c0 < n_new; c0 += SCAN_CHUNK) {
    const int n = min(SCAN_CHUNK, n_new - c0);
    __syncthreads();                            // the chunk before has been read
    for (int idx = threadIdx.x; idx < n * N; idx += blockDim.x) {
      const int tt = idx / N, nn = idx % N;
      const T* brow = a.bc + (size_t)(row0 + c0 + tt) * a.ldbc;
      bc_s[(tt * 2 + 0) * N + nn] = mi::to_float(brow[a.b_off + nn]);
      bc_s[(tt * 2 + 1) * N + nn] = mi::to_float(brow[a.c_off + nn]);
    }
    float dtv[SCAN_CHUNK], uv[SCAN_CHUNK], zv[SCAN_CHUNK];
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
      const size_t t = (size_t)(row0 + c0 + min(tt, n - 1));
      dtv[tt] = mi::to_float(a.dt_in[t * a.lddt + cc]);
      uv[tt] = mi::to_float(a.u[t * a.ldu + cc]);
      zv[tt] = mi::to_float(a.z[t * a.ldz + cc]);
    }
    __syncthreads();
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
      if (tt < n) {
        const float dt = softplus_f(dtv[tt] + dtb);
        const float u = uv[tt];
        const float du = dt * u;
        const float* Bv = bc_s + (tt * 2 + 0) * N;
        const float* Cv = bc_s + (tt * 2 + 1) * N;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
          const int nn = part * SPT + i;
          if (nn < N) {
            S[i] = fmaf(expf(dt * A[i]), S[i], du * Bv[nn]);
            acc = fmaf(S[i], Cv[nn], acc);
          }
        }
        for (int o = a.P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (live && part == 0)
          a.y[(size_t)(row0 + c0 + tt) * a.ldy + cc] = mi::from_float<T>((acc + Dc * u) * silu_f(zv[tt]));
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      const int n = part * SPT + i;
      if (n < a.N) st[n] = S[i];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// Gated delta rule.  Per head, with the state S [dim, vdim], token after token:
//   qh = q / sqrt(sum q^2 + 1e-6) * dim^-1/2,  kh = k / sqrt(sum k^2 + 1e-6)       (q, k of the head's q/k head)
//   g[i] = exp(-exp(A_log[head]) * softplus(a[t, head, i] + dt_bias[head, i])),    beta = sigmoid(b[t, head])
//   S[i, :] <- g[i] * S[i, :];   u = beta * (v - S^T kh);   S <- S + kh u^T;   o = S^T qh
//   out[t, head, :] = o / sqrt(mean(o^2) + eps) * norm_w * sigmoid(gate[t, head, :])
// A block per (item, head).  Thread (j, r) keeps rows r * DK .. r * DK + DK - 1 of column j of S in registers; the R
// threads of a column are neighbouring lanes.  The tokens go through shared memory in chunks: the chunk's q, k, decays,
// values and betas are prepared by all threads (a warp per token for the unit norms), then the recurrence runs over the
// chunk, then the chunk's outputs are normalised and gated (a warp per token).
template <typename T>
struct DeltaArgs {
  T* out; int ldo;                       // [tokens, heads * vdim]
  const T* q; const T* k; int ldqk;      // rows of the convolved q and k: head g at column g * dim
  const T* v; int ldv;                   // head h at column h * vdim
  const T* a; int lda;                   // decay input, head h at column h * dim
  const T* b; int ldb;                   // beta logits, head h at column h
  const T* gate; int ldg;                // output gate logits, head h at column h * vdim
  const float* dt_bias; const float* A_log; const float* norm_w;
  float* state; long long state_stride;  // [slot][heads][dim][vdim]
  const int* q_start; const int* q_len; const int* seq_slot;
  int heads, kv_heads, dim, vdim, R, chunk;
  float eps;
};

__device__ __forceinline__ int pad_idx(int i) { return i + (i >> 5); }

constexpr int delta_max_threads(int dk) { return dk <= 16 ? 1024 : dk <= 64 ? 512 : 256; }

template <typename T, int DK>
__global__ void __launch_bounds__(delta_max_threads(DK))
gated_delta_kernel(DeltaArgs<T> a) {
  extern __shared__ float sm[];
  const int item = blockIdx.y, head = blockIdx.x;
  const int kvh = head / (a.heads / a.kv_heads);
  const int row0 = a.q_start[item], n_new = a.q_len[item], slot = a.seq_slot[item];
  const int R = a.R, dim = a.dim, vdim = a.vdim;
  const int col = threadIdx.x / R, r = threadIdx.x % R;
  const bool live = col < vdim;
  const int dpad = pad_idx(dim) + 1;
  // per chunk token: q [dpad], k [dpad], g [dpad], v / out [vdim], beta
  const int tok_floats = 3 * dpad + vdim + 1;
  const float neg_rate = -expf(a.A_log[head]);
  mi::grid_dependency_sync();
  float* st = a.state + (size_t)slot * a.state_stride + (size_t)head * dim * vdim;
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const int row = r * DK + i;
    S[i] = (live && row < dim) ? st[(size_t)row * vdim + col] : 0.f;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const float q_scale = rsqrtf((float)dim);
  for (int c0 = 0; c0 < n_new; c0 += a.chunk) {
    const int n = min(a.chunk, n_new - c0);
    __syncthreads();
    // ---- the chunk's inputs
    for (int idx = threadIdx.x; idx < n * dim; idx += blockDim.x) {
      const int tt = idx / dim, i = idx % dim;
      const size_t t = (size_t)(row0 + c0 + tt);
      float* base = sm + (size_t)tt * tok_floats;
      base[pad_idx(i)] = mi::to_float(a.q[t * a.ldqk + kvh * dim + i]);
      base[dpad + pad_idx(i)] = mi::to_float(a.k[t * a.ldqk + kvh * dim + i]);
      const float z = mi::to_float(a.a[t * a.lda + head * dim + i]) + a.dt_bias[head * dim + i];
      base[2 * dpad + pad_idx(i)] = expf(neg_rate * softplus_f(z));
    }
    for (int idx = threadIdx.x; idx < n * vdim; idx += blockDim.x) {
      const int tt = idx / vdim, jv = idx % vdim;
      const size_t t = (size_t)(row0 + c0 + tt);
      sm[(size_t)tt * tok_floats + 3 * dpad + jv] = mi::to_float(a.v[t * a.ldv + head * vdim + jv]);
    }
    for (int tt = threadIdx.x; tt < n; tt += blockDim.x)
      sm[(size_t)tt * tok_floats + 3 * dpad + vdim] = sigmoid_f(mi::to_float(a.b[(size_t)(row0 + c0 + tt) * a.ldb + head]));
    __syncthreads();
    for (int tt = warp; tt < n; tt += warps) {
      float* base = sm + (size_t)tt * tok_floats;
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < dim; i += 32) {
        const float x = base[pad_idx(i)], y = base[dpad + pad_idx(i)];
        sq = fmaf(x, x, sq);
        sk = fmaf(y, y, sk);
      }
      sq = mi::warp_sum(sq);
      sk = mi::warp_sum(sk);
      const float fq = q_scale / sqrtf(sq + 1e-6f), fk = 1.f / sqrtf(sk + 1e-6f);
      for (int i = lane; i < dim; i += 32) {
        base[pad_idx(i)] *= fq;
        base[dpad + pad_idx(i)] *= fk;
      }
    }
    __syncthreads();
    // ---- the recurrence over the chunk
    for (int tt = 0; tt < n; ++tt) {
      float* base = sm + (size_t)tt * tok_floats;
      const float* qv = base;
      const float* kv = base + dpad;
      const float* gv = base + 2 * dpad;
      float ks = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        const int row = r * DK + i;
        if (row < dim) {
          S[i] *= gv[pad_idx(row)];
          ks = fmaf(kv[pad_idx(row)], S[i], ks);
        }
      }
      for (int o = R >> 1; o > 0; o >>= 1) ks += __shfl_xor_sync(0xffffffffu, ks, o);
      const float vj = live ? base[3 * dpad + col] : 0.f;
      const float u = base[3 * dpad + vdim] * (vj - ks);
      float oj = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        const int row = r * DK + i;
        if (row < dim) {
          S[i] = fmaf(kv[pad_idx(row)], u, S[i]);
          oj = fmaf(qv[pad_idx(row)], S[i], oj);
        }
      }
      for (int o = R >> 1; o > 0; o >>= 1) oj += __shfl_xor_sync(0xffffffffu, oj, o);
      // the value's place is free once every thread of the column has read it: all R of them sit in this warp
      __syncwarp();
      if (live && r == 0) base[3 * dpad + col] = oj;
    }
    __syncthreads();
    // ---- the chunk's outputs: unit root mean square over the head, weight, gate
    for (int tt = warp; tt < n; tt += warps) {
      const float* o = sm + (size_t)tt * tok_floats + 3 * dpad;
      const size_t t = (size_t)(row0 + c0 + tt);
      float ss = 0.f;
      for (int jv = lane; jv < vdim; jv += 32) ss = fmaf(o[jv], o[jv], ss);
      ss = mi::warp_sum(ss);
      const float rstd = 1.f / sqrtf(ss / (float)vdim + a.eps);
      for (int jv = lane; jv < vdim; jv += 32) {
        const float gl = mi::to_float(a.gate[t * a.ldg + head * vdim + jv]);
        a.out[t * a.ldo + head * vdim + jv] = mi::from_float<T>(o[jv] * rstd * a.norm_w[jv] * sigmoid_f(gl));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    const int row = r * DK + i;
    if (live && row < dim) st[(size_t)row * vdim + col] = S[i];
  }
}

}  // namespace

MI_API int mi_causal_conv(void* out, int ldo, const void* x, int ldx, int dtype, const float* w, const float* bias,
                          float* state, long long state_stride, const int* token_item, const int* q_start, const int* q_len,
                          const int* seq_slot, int T, int items, int C, int taps, int silu, cudaStream_t stream) {
  MI_REQUIRE(T >= 0 && items >= 0 && C > 0 && taps >= 1 && taps <= MAX_TAPS, "causal_conv: bad sizes C=%d taps=%d (taps up to %d)", C, taps, MAX_TAPS);
  MI_REQUIRE(T <= 65535 && items <= 65535, "causal_conv: more than 65535 tokens or items in one launch");
  MI_REQUIRE(state_stride >= (long long)(taps - 1) * C, "causal_conv: the state rows are too short");
  if (T == 0) return 0;
  dim3 grid((C + 255) / 256, T), sgrid((C + 255) / 256, items);
  if (dtype == MI_BF16) {
    mi::launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)x, ldx, w, bias,
               (const float*)state, state_stride, token_item, q_start, seq_slot, C, taps, silu);
    if (taps > 1) mi::launch(conv_state_kernel<__nv_bfloat16>, sgrid, dim3(256), 0, stream, state, state_stride, (const __nv_bfloat16*)x, ldx,
                             q_start, q_len, seq_slot, C, taps);
  } else if (dtype == MI_F32) {
    mi::launch(causal_conv_kernel<float>, grid, dim3(256), 0, stream, (float*)out, ldo, (const float*)x, ldx, w, bias,
               (const float*)state, state_stride, token_item, q_start, seq_slot, C, taps, silu);
    if (taps > 1) mi::launch(conv_state_kernel<float>, sgrid, dim3(256), 0, stream, state, state_stride, (const float*)x, ldx,
                             q_start, q_len, seq_slot, C, taps);
  } else {
    return mi_fail("causal_conv: unknown dtype %d", dtype);
  }
  MI_LAUNCH_OK("causal_conv");
  return 0;
}

MI_API int mi_selective_scan(void* y, int ldy, const void* u, int ldu, const void* dt_in, int lddt, const void* bc, int ldbc,
                             int b_off, int c_off, const void* z, int ldz, int dtype, const float* dt_bias, const float* A_log,
                             const float* D, float* state, long long state_stride, const int* q_start, const int* q_len,
                             const int* seq_slot, int items, int inner, int N, cudaStream_t stream) {
  MI_REQUIRE(items >= 0 && items <= 65535 && inner > 0 && N > 0 && N <= 32 * SPT, "selective_scan: bad sizes inner=%d state=%d (state up to %d)", inner, N, 32 * SPT);
  MI_REQUIRE(state_stride >= (long long)inner * N, "selective_scan: the state rows are too short");
  if (items == 0) return 0;
  int P = 1;
  while (P * SPT < N) P *= 2;
  const int per_block = SCAN_THREADS / P;
  const size_t smem = (size_t)SCAN_CHUNK * 2 * N * sizeof(float);
  dim3 grid((inner + per_block - 1) / per_block, items);
#define MI_SCAN(TT)                                                                                               \
  do {                                                                                                            \
    ScanArgs<TT> a;                                                                                               \
    a.y = (TT*)y; a.ldy = ldy; a.u = (const TT*)u; a.ldu = ldu; a.dt_in = (const TT*)dt_in; a.lddt = lddt;        \
    a.bc = (const TT*)bc; a.ldbc = ldbc; a.b_off = b_off; a.c_off = c_off; a.z = (const TT*)z; a.ldz = ldz;       \
    a.dt_bias = dt_bias; a.A_log = A_log; a.D = D; a.state = state; a.state_stride = state_stride;                \
    a.q_start = q_start; a.q_len = q_len; a.seq_slot = seq_slot; a.inner = inner; a.N = N; a.P = P;               \
    mi::launch(selective_scan_kernel<TT>, grid, dim3(SCAN_THREADS), smem, stream, a);                                         \
  } while (0)
  if (dtype == MI_BF16) MI_SCAN(__nv_bfloat16);
  else if (dtype == MI_F32) MI_SCAN(float);
  else return mi_fail("selective_scan: unknown dtype %d", dtype);
#undef MI_SCAN
  MI_LAUNCH_OK("selective_scan");
  return 0;
}

MI_API int mi_gated_delta(void* out, int ldo, const void* q, const void* k, int ldqk, const void* v, int ldv, const void* a_in, int lda,
                          const void* b_in, int ldb, const void* gate, int ldg, int dtype, const float* dt_bias, const float* A_log,
                          const float* norm_w, float eps, float* state, long long state_stride, const int* q_start, const int* q_len,
                          const int* seq_slot, int items, int heads, int kv_heads, int dim, int vdim, cudaStream_t stream) {
  MI_REQUIRE(items >= 0 && items <= 65535 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "gated_delta: bad head counts %d / %d", heads, kv_heads);
  MI_REQUIRE(dim > 0 && vdim > 0 && vdim <= 1024 && dim <= 4096, "gated_delta: bad sizes dim=%d vdim=%d", dim, vdim);
  MI_REQUIRE(state_stride >= (long long)heads * dim * vdim, "gated_delta: the state rows are too short");
  if (items == 0) return 0;
  // rows of a column a thread keeps (DK) and threads a column (R, a power of two up to 32): the smallest DK whose block
  // fits, so that a thread's share of the state stays in registers
  int DK = 0, R = 1;
  for (int dk = 16; dk <= 128 && !DK; dk *= 2) {
    int r = 1;
    while (r * dk < dim) r *= 2;
    if (r <= 32 && ((vdim * r + 31) / 32) * 32 <= delta_max_threads(dk)) { DK = dk; R = r; }
  }
  MI_REQUIRE(DK > 0, "gated_delta: a state of %d x %d values a head does not fit a block's registers", dim, vdim);
  const int threads = ((vdim * R + 31) / 32) * 32;
  const int dpad = dim + (dim >> 5) + 1;
  const int tok_floats = 3 * dpad + vdim + 1;
  int chunk = (40 * 1024 / 4) / tok_floats;
  if (chunk > 32) chunk = 32;
  MI_REQUIRE(chunk >= 1, "gated_delta: a token's vectors do not fit shared memory");
  const size_t smem = (size_t)chunk * tok_floats * sizeof(float);
#define MI_DELTA(TT, DKV)                                                                                         \
  do {                                                                                                            \
    DeltaArgs<TT> d;                                                                                              \
    d.out = (TT*)out; d.ldo = ldo; d.q = (const TT*)q; d.k = (const TT*)k; d.ldqk = ldqk; d.v = (const TT*)v; d.ldv = ldv; \
    d.a = (const TT*)a_in; d.lda = lda; d.b = (const TT*)b_in; d.ldb = ldb; d.gate = (const TT*)gate; d.ldg = ldg; \
    d.dt_bias = dt_bias; d.A_log = A_log; d.norm_w = norm_w; d.state = state; d.state_stride = state_stride;      \
    d.q_start = q_start; d.q_len = q_len; d.seq_slot = seq_slot; d.heads = heads; d.kv_heads = kv_heads; d.dim = dim; \
    d.vdim = vdim; d.R = R; d.chunk = chunk; d.eps = eps;                                                         \
    mi::launch(gated_delta_kernel<TT, DKV>, dim3(heads, items), dim3(threads), smem, stream, d);                  \
  } while (0)
#define MI_DELTA_DK(TT)                 \
  do {                                  \
    if (DK == 16) MI_DELTA(TT, 16);     \
    else if (DK == 32) MI_DELTA(TT, 32); \
    else if (DK == 64) MI_DELTA(TT, 64); \
    else MI_DELTA(TT, 128);             \
  } while (0)
  if (dtype == MI_BF16) MI_DELTA_DK(__nv_bfloat16);
  else if (dtype == MI_F32) MI_DELTA_DK(float);
  else return mi_fail("gated_delta: unknown dtype %d", dtype);
#undef MI_DELTA_DK
#undef MI_DELTA
  MI_LAUNCH_OK("gated_delta");
  return 0;
}
