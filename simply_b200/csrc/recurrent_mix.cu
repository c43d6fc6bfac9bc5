// Kernels of the recurrent mixers: the gated delta rule with its short convolutions, the
// forget-gate recurrence, and the mean of RMS-normed branches.  Everything here computes in float32; T is the storage type of
// the activations that come in from and go out to matrix products.
//
//   inputs    y_c[t] = silu(sum_j w[c, j] x_c[t - (taps-1) + j])   x before the request's start is
//                                                                   0, before the step's start it
//                                                                   comes from the request's state
//             q, k   = y / sqrt(sum_head y^2 + 1e-6)   (q also times head_dim^-1/2)
//             beta   = sigmoid(b),  g = exp(-exp(A) * softplus(a + dt))
//   scan      S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   output    o / sqrt(mean_head o^2 + eps) * w * sigmoid(gate)
//   mean      (1/n) sum_i x_i / sqrt(mean x_i^2 + eps) * w_i
#include "common.cuh"

#define SB_ERR_BAD_SLOT 16  // a state slot outside the state tensor

// A decode graph pads its batch by repeating the last request: only the first row of a slot
// may write the slot's state (the others compute results that are dropped).
__device__ __forceinline__ bool first_row_of_slot(const int* slots, int b) {
  const int slot = slots[b];
  for (int i = 0; i < b; ++i)
    if (slots[i] == slot) return false;
  return true;
}

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------
// Inputs of the delta rule.  One block per token.
//   pre  [T, pre_width]: q | k | v | b   (q, k: G heads of d; v: H heads of dv; b: H)
//   low  [T, low_width]: a (H * d) | ...
//   conv_state [slots, taps - 1, C] float32, C = 2 G d + H dv
// ---------------------------------------------------------------------------
// TAPS > 0: the number of taps at compile time, so that a channel's loads go out together.
template <typename T, int TAPS>
__global__ void __launch_bounds__(512)
delta_inputs_kernel(const T* __restrict__ pre, int pre_width, const T* __restrict__ low, int low_width,
                    const float* __restrict__ conv_w, const float* __restrict__ conv_state,
                    const float* __restrict__ dt_bias, const float* __restrict__ neg_rate,
                    const int* __restrict__ token_seq, const int* __restrict__ cu_q, const int* __restrict__ slots,
                    int num_slots, int taps, int G, int H, int d, int dv,
                    float* __restrict__ q_out, float* __restrict__ k_out, float* __restrict__ v_out,
                    float* __restrict__ decay_out, float* __restrict__ beta_out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  extern __shared__ float y[];  // C floats
  const int t = blockIdx.x;
  const int b = token_seq[t];
  const int first = cu_q[b];
  const int i = t - first;
  int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    slot = 0;
  }
  const int qk = G * d, C = 2 * qk + H * dv;
  const float* state = conv_state + (size_t)slot * (taps - 1) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    if (TAPS > 0) {
      float x[TAPS > 0 ? TAPS : 1], w[TAPS > 0 ? TAPS : 1];
#pragma unroll
      for (int j = 0; j < TAPS; ++j) {
        const int idx = i - (TAPS - 1) + j;
        x[j] = idx >= 0 ? to_f32<T>(pre[(size_t)(first + idx) * pre_width + c])
                        : state[(size_t)(TAPS - 1 + idx) * C + c];
        w[j] = conv_w[(size_t)c * TAPS + j];
      }
#pragma unroll
      for (int j = 0; j < TAPS; ++j) acc = fmaf(w[j], x[j], acc);
    } else {
      for (int j = 0; j < taps; ++j) {
        const int idx = i - (taps - 1) + j;
        const float x = idx >= 0 ? to_f32<T>(pre[(size_t)(first + idx) * pre_width + c])
                                 : state[(size_t)(taps - 1 + idx) * C + c];
        acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
      }
    }
    y[c] = acc * sigmoid_f32(acc);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float q_scale = 1.0f / sqrtf((float)d);
  for (int head = warp; head < 2 * G; head += nwarps) {  // q heads, then k heads
    const float* src = y + (size_t)head * d;
    float ss = 0.f;
    for (int c = lane; c < d; c += 32) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    float scale = 1.0f / sqrtf(ss + 1e-6f);
    float* dst;
    if (head < G) {
      scale *= q_scale;
      dst = q_out + ((size_t)t * G + head) * d;
    } else {
      dst = k_out + ((size_t)t * G + (head - G)) * d;
    }
    for (int c = lane; c < d; c += 32) dst[c] = src[c] * scale;
  }
  for (int c = threadIdx.x; c < H * dv; c += blockDim.x) v_out[(size_t)t * H * dv + c] = y[2 * qk + c];
  for (int h = threadIdx.x; h < H; h += blockDim.x)
    beta_out[(size_t)t * H + h] = sigmoid_f32(to_f32<T>(pre[(size_t)t * pre_width + C + h]));
  for (int c = threadIdx.x; c < H * d; c += blockDim.x) {
    const float a = to_f32<T>(low[(size_t)t * low_width + c]) + dt_bias[c];
    decay_out[(size_t)t * H * d + c] = expf(neg_rate[c / d] * softplus_f32(a));
  }
}

// The convolution's state after the step: the last taps - 1 inputs of (state, new inputs).  One
// thread per (sequence, channel), ascending, so that it reads only what it has not yet written.
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ pre, int pre_width, float* __restrict__ conv_state,
                                  const int* __restrict__ cu_q, const int* __restrict__ slots, int num_slots,
                                  int taps, int C) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = slots[b];
  if (c >= C || slot < 0 || slot >= num_slots || !first_row_of_slot(slots, b)) return;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  float* state = conv_state + (size_t)slot * (taps - 1) * C;
  for (int r = 0; r < taps - 1; ++r) {
    const int idx = n - (taps - 1) + r;
    state[(size_t)r * C + c] = idx >= 0 ? to_f32<T>(pre[(size_t)(first + idx) * pre_width + c])
                                        : state[(size_t)(taps - 1 + idx) * C + c];
  }
}

extern "C" int sb_delta_inputs(const void* pre, int pre_width, const void* low, int low_width, int dtype,
                               const float* conv_w, float* conv_state, const float* dt_bias,
                               const float* neg_rate, const int* token_seq, const int* cu_q, const int* slots,
                               int num_tokens, int num_seqs, int num_slots, int taps, int G, int H, int d, int dv,
                               float* q_out, float* k_out, float* v_out, float* decay_out, float* beta_out,
                               int* err, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int C = 2 * G * d + H * dv;
  const size_t smem = (size_t)C * sizeof(float);
  if (taps < 1 || G <= 0 || H % G || smem > 200 * 1024) return -13;
#define SB_DELTA_INPUTS(T_, TAPS_)                                                                             \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(delta_inputs_kernel<T_, TAPS_>, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                           (int)smem);                                                                         \
    sb_launch(delta_inputs_kernel<T_, TAPS_>, num_tokens, 512, smem, stream, (const T_*)pre, pre_width,        \
              (const T_*)low, low_width, conv_w, (const float*)conv_state, dt_bias, neg_rate, token_seq, cu_q, \
              slots, num_slots, taps, G, H, d, dv, q_out, k_out, v_out, decay_out, beta_out, err);             \
  } while (0)
#define SB_DELTA_INPUTS_T(T_)                    \
  do {                                           \
    if (taps == 4) SB_DELTA_INPUTS(T_, 4);       \
    else if (taps == 3) SB_DELTA_INPUTS(T_, 3);  \
    else if (taps == 2) SB_DELTA_INPUTS(T_, 2);  \
    else SB_DELTA_INPUTS(T_, 0);                 \
  } while (0)
  if (dtype == SB_DTYPE_F32) SB_DELTA_INPUTS_T(float);
  else SB_DELTA_INPUTS_T(bf16);
#undef SB_DELTA_INPUTS_T
#undef SB_DELTA_INPUTS
  SB_LAUNCH_CHECK();
  if (taps > 1) {
    const dim3 grid((C + 127) / 128, num_seqs);
    if (dtype == SB_DTYPE_F32)
      sb_launch(conv_state_kernel<float>, grid, 128, 0, stream, (const float*)pre, pre_width, conv_state, cu_q,
                slots, num_slots, taps, C);
    else
      sb_launch(conv_state_kernel<bf16>, grid, 128, 0, stream, (const bf16*)pre, pre_width, conv_state, cu_q,
                slots, num_slots, taps, C);
    SB_LAUNCH_CHECK();
  }
  return 0;
}

// ---------------------------------------------------------------------------
// The scan.  A block owns `cols` value columns of one (sequence, head) and walks the sequence's
// tokens of this step in order.  A column of S is held by RS neighbouring lanes, each with the
// rows rs, rs + RS, ... (ROWS of them) in registers; the two sums over rows per token are
// butterfly sums over those lanes, in an order that does not depend on the step's shape.  A
// token is a chain of dependent instructions, and a sequence has only heads * value_dim columns to
// work on side by side: few rows per thread (8, a column over up to 32 lanes) keep the chain
// short and give the SMs several warps each, which is what the walk's time hangs on (with 32 rows
// per thread a 2,048-token prompt took 1 microsecond per token, one warp per scheduler, every
// instruction's latency in the open).  k, q,
// g, v and beta of SCAN_CHUNK tokens at a time come to shared memory by cp.async, the next
// chunk while the block works on this one.
// ---------------------------------------------------------------------------
#define SCAN_CHUNK chunk  // tokens per fetch: a kernel argument (the buffers' layout depends on it)
#define SCAN_ROWS 32

__device__ __forceinline__ void scan_copy4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void scan_copy16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem));
}

// VEC (head_dim a multiple of 4): a thread's rows are the groups of four 4 (rs + RS r) .. + 3, read
// from shared memory as float4, with one partial sum per row of a group, so that a token's two
// sums are four chains of eight instead of one of thirty-two.
template <int RS, int ROWS, bool VEC>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  const float* __restrict__ decay, const float* __restrict__ beta, float* __restrict__ state,
                  const int* __restrict__ cu_q, const int* __restrict__ slots, int num_slots, int G, int H, int d,
                  int dv, int cols, int chunk, float* __restrict__ out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  // Two buffers of: k [CHUNK][d], q [CHUNK][d], g [CHUNK][d], v [CHUNK][cols], beta [CHUNK].
  extern __shared__ __align__(16) float stage[];
  const int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * cols;
  const int rs = threadIdx.x % RS, col_local = threadIdx.x / RS;
  const int col = col0 + col_local;
  const bool on = col_local < cols && col < dv;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    return;
  }
  const int g_head = h / (H / G);
  const int cols_pad = (cols + 3) & ~3;
  const int buffer = SCAN_CHUNK * (3 * d + cols_pad + 4);
  const bool vec = (d & 3) == 0;
  // When a row's 16-byte pieces divide the block: a fixed piece per thread, rows dealt out in turn.
  const int pieces = d >> 2;
  const int copy_rows = (vec && pieces <= (int)blockDim.x && blockDim.x % pieces == 0) ? blockDim.x / pieces : 0;
  const int copy_row = copy_rows ? threadIdx.x / pieces : 0, copy_c = copy_rows ? (threadIdx.x % pieces) * 4 : 0;

  auto issue = [&](int which, int base) {
    float* buf = stage + which * buffer;
    const int count = min(SCAN_CHUNK, n - base);
    if (vec && copy_rows > 0) {
      // thread (copy_row, copy_c) of every pass copies 16 bytes of one of the chunk's 3 * count rows
      for (int row = copy_row; row < 3 * count; row += copy_rows) {
        const int i = row / 3, kind = row - 3 * i;
        const size_t t = (size_t)(first + base + i);
        const float* src = kind == 0 ? k + (t * G + g_head) * d : kind == 1 ? q + (t * G + g_head) * d
                                                                             : decay + (t * H + h) * d;
        scan_copy16(buf + (kind * SCAN_CHUNK + i) * d + copy_c, src + copy_c);
      }
    } else if (vec) {
      const int d4 = d >> 2;
      for (int idx = threadIdx.x; idx < count * 3 * d4; idx += blockDim.x) {
        const int i = idx / (3 * d4), rem = idx - i * 3 * d4, kind = rem / d4, c = (rem - kind * d4) * 4;
        const size_t t = (size_t)(first + base + i);
        const float* src = kind == 0 ? k + (t * G + g_head) * d : kind == 1 ? q + (t * G + g_head) * d
                                                                             : decay + (t * H + h) * d;
        scan_copy16(buf + (kind * SCAN_CHUNK + i) * d + c, src + c);
      }
    } else {
      for (int idx = threadIdx.x; idx < count * 3 * d; idx += blockDim.x) {
        const int i = idx / (3 * d), rem = idx - i * 3 * d, kind = rem / d, c = rem - kind * d;
        const size_t t = (size_t)(first + base + i);
        const float* src = kind == 0 ? k + (t * G + g_head) * d : kind == 1 ? q + (t * G + g_head) * d
                                                                             : decay + (t * H + h) * d;
        scan_copy4(buf + (kind * SCAN_CHUNK + i) * d + c, src + c);
      }
    }
    float* bv = buf + 3 * SCAN_CHUNK * d;
    for (int idx = threadIdx.x; idx < count * cols; idx += blockDim.x) {
      const int i = idx / cols, c = idx - i * cols;
      scan_copy4(bv + i * cols_pad + c, v + ((size_t)(first + base + i) * H + h) * dv + min(col0 + c, dv - 1));
    }
    float* bb = bv + SCAN_CHUNK * cols_pad;
    for (int i = threadIdx.x; i < count; i += blockDim.x) scan_copy4(bb + i, beta + (size_t)(first + base + i) * H + h);
    asm volatile("cp.async.commit_group;\n" ::);
  };

  if (n > 0) issue(0, 0);
  float* S = state + ((size_t)slot * H + h) * d * dv;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = VEC ? 4 * (rs + RS * (r >> 2)) + (r & 3) : rs + RS * r;
    s[r] = (on && row < d) ? S[(size_t)row * dv + col] : 0.f;
  }
  int which = 0;
  for (int base = 0; base < n; base += SCAN_CHUNK, which ^= 1) {
    const int count = min(SCAN_CHUNK, n - base);
    if (base + SCAN_CHUNK < n) {
      issue(which ^ 1, base + SCAN_CHUNK);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* buf = stage + which * buffer;
    for (int i = 0; i < count; ++i) {
      const float* kk = buf + i * d;
      const float* qq = buf + (SCAN_CHUNK + i) * d;
      const float* gg = buf + (2 * SCAN_CHUNK + i) * d;
      const float vv = buf[3 * SCAN_CHUNK * d + i * cols_pad + min(col_local, cols - 1)];
      const float bb = buf[3 * SCAN_CHUNK * d + SCAN_CHUNK * cols_pad + i];
      float dot = 0.f, od = 0.f;
      if constexpr (VEC) {
        // One pass over the decayed state gives both sums: with S' = diag(g) S, the result after the
        // write is S'^T q + u (k . q), so it needs no second pass after u is known.
        float4 k4[ROWS / 4];
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f, kq = 0.f;
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const int at = rs + RS * r;
          if (4 * at < d) {
            const float4 g4 = reinterpret_cast<const float4*>(gg)[at];
            const float4 q4 = reinterpret_cast<const float4*>(qq)[at];
            k4[r] = reinterpret_cast<const float4*>(kk)[at];
            s[4 * r] *= g4.x; d0 = fmaf(s[4 * r], k4[r].x, d0); o0 = fmaf(s[4 * r], q4.x, o0);
            s[4 * r + 1] *= g4.y; d1 = fmaf(s[4 * r + 1], k4[r].y, d1); o1 = fmaf(s[4 * r + 1], q4.y, o1);
            s[4 * r + 2] *= g4.z; d2 = fmaf(s[4 * r + 2], k4[r].z, d2); o2 = fmaf(s[4 * r + 2], q4.z, o2);
            s[4 * r + 3] *= g4.w; d3 = fmaf(s[4 * r + 3], k4[r].w, d3); o3 = fmaf(s[4 * r + 3], q4.w, o3);
            kq = fmaf(k4[r].x, q4.x, fmaf(k4[r].y, q4.y, fmaf(k4[r].z, q4.z, fmaf(k4[r].w, q4.w, kq))));
          }
        }
        dot = (d0 + d1) + (d2 + d3);
        od = (o0 + o1) + (o2 + o3);
#pragma unroll
        for (int o = 1; o < RS; o <<= 1) {
          dot += __shfl_xor_sync(0xffffffffu, dot, o);
          od += __shfl_xor_sync(0xffffffffu, od, o);
          kq += __shfl_xor_sync(0xffffffffu, kq, o);
        }
        const float u = bb * (vv - dot);
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const int at = rs + RS * r;
          if (4 * at < d) {
            s[4 * r] = fmaf(k4[r].x, u, s[4 * r]);
            s[4 * r + 1] = fmaf(k4[r].y, u, s[4 * r + 1]);
            s[4 * r + 2] = fmaf(k4[r].z, u, s[4 * r + 2]);
            s[4 * r + 3] = fmaf(k4[r].w, u, s[4 * r + 3]);
          }
        }
        od = fmaf(u, kq, od);
      } else {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const int row = rs + RS * r;
          if (row < d) {
            s[r] *= gg[row];
            dot = fmaf(s[r], kk[row], dot);
          }
        }
#pragma unroll
        for (int o = 1; o < RS; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float u = bb * (vv - dot);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const int row = rs + RS * r;
          if (row < d) {
            s[r] = fmaf(kk[row], u, s[r]);
            od = fmaf(s[r], qq[row], od);
          }
        }
#pragma unroll
        for (int o = 1; o < RS; o <<= 1) od += __shfl_xor_sync(0xffffffffu, od, o);
      }
      if (on && rs == 0) out[((size_t)(first + base + i) * H + h) * dv + col] = od;
    }
    __syncthreads();  // the buffer is filled again two chunks on
  }
  if (on && first_row_of_slot(slots, b)) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = VEC ? 4 * (rs + RS * (r >> 2)) + (r & 3) : rs + RS * r;
      if (row < d) S[(size_t)row * dv + col] = s[r];
    }
  }
}

extern "C" int sb_delta_scan(const float* q, const float* k, const float* v, const float* decay, const float* beta,
                             float* state, const int* cu_q, const int* slots, int num_seqs, int num_slots, int G,
                             int H, int d, int dv, int max_q_len, float* out, int* err, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (d <= 0 || d > 32 * SCAN_ROWS || dv <= 0 || G <= 0 || H % G) return -13;
  // Rows per thread: 8 where the head allows (a column over at most 32 lanes), else 32.
  const bool vec = d % 4 == 0;
  const int rows = (vec && d <= 8 * 32) ? 8 : SCAN_ROWS;
  int rs = 1;
  while (rs * rows < d) rs <<= 1;
  // Long walks: blocks of 128 threads even when that leaves SMs without one (every block fetches its
  // head's k, q and g, so narrower blocks fetch them more often) and chunks of 16 tokens (a
  // 2,048-token prompt of 16 heads: 0.84 ms; 0.90 with chunks of 8; 1.02 with 64 threads).  Steps of
  // a few tokens read and write the state and little else: narrow blocks with small buffers, many
  // to an SM.
  const bool long_walk = max_q_len >= 64;
  const int threads = long_walk ? 128 : 64;
  int chunk = 1;
  while (chunk < 16 && chunk < max_q_len) chunk <<= 1;
  if (long_walk && (size_t)2 * 16 * (3 * d + 36) * sizeof(float) > 200 * 1024) chunk = 8;
  int cols = threads / rs;
  if (cols < 1) cols = 1;
  if (cols > dv) cols = dv;
  const int block = ((cols * rs + 31) / 32) * 32;
  const dim3 grid(H, num_seqs, (dv + cols - 1) / cols);
  const size_t smem = (size_t)2 * SCAN_CHUNK * (3 * d + ((cols + 3) & ~3) + 4) * sizeof(float);
  if (smem > 200 * 1024) return -13;
#define SB_SCAN_V(RS_, ROWS_, VEC_)                                                                           \
  do {                                                                                                        \
    if (smem > 48 * 1024)                                                                                     \
      cudaFuncSetAttribute(delta_scan_kernel<RS_, ROWS_, VEC_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                                        \
    if (long_walk)                                                                                            \
      sb_launch_plain(delta_scan_kernel<RS_, ROWS_, VEC_>, grid, block, smem, stream, q, k, v, decay, beta,   \
                      state, cu_q, slots, num_slots, G, H, d, dv, cols, chunk, out, err);                     \
    else                                                                                                      \
      sb_launch(delta_scan_kernel<RS_, ROWS_, VEC_>, grid, block, smem, stream, q, k, v, decay, beta, state, \
                cu_q, slots, num_slots, G, H, d, dv, cols, chunk, out, err);                                  \
  } while (0)
#define SB_SCAN(RS_)                                  \
  do {                                                \
    if (rows == 8) SB_SCAN_V(RS_, 8, true);           \
    else if (vec) SB_SCAN_V(RS_, SCAN_ROWS, true);    \
    else SB_SCAN_V(RS_, SCAN_ROWS, false);            \
  } while (0)
  switch (rs) {
    case 1: SB_SCAN(1); break;
    case 2: SB_SCAN(2); break;
    case 4: SB_SCAN(4); break;
    case 8: SB_SCAN(8); break;
    case 16: SB_SCAN(16); break;
    default: SB_SCAN(32); break;
  }
#undef SB_SCAN
#undef SB_SCAN_V
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// The forget-gate recurrence (HGRN2): per head a matrix S [d, dv] whose rows decay by f and take in
// (1 - f) v, read by q after the write:
//   q = silu(pq),  f = l + (1 - l) sigmoid(pf + b),  S <- diag(f) S + (1 - f) v^T,  o = S^T q
// `pre` [T, row_width] holds pq (H d) | pf (H d) | v (H dv) as the projection left them.  Two
// kernels: the inputs (activations and gates once per token, float32: qf [T, 2, H d] and v [T, H dv]),
// and the walk, whose layout is the delta rule's: a column of S over RS neighbouring lanes with ROWS
// rows each, a block per (head, sequence, tile of columns), q, f and v of 16 tokens at a time
// by cp.async with the next chunk under way, the state written back by the slot's first row.  The
// state's update is one multiply-add per row and token and does not wait for the sum that reads it.
// ---------------------------------------------------------------------------
#define FORGET_CHUNK 16
#define FORGET_TOGETHER 8  // tokens whose updates and sums are interleaved (divides the chunk)

template <typename T>
__global__ void __launch_bounds__(256)
forget_inputs_kernel(const T* __restrict__ pre, int row_width, const float* __restrict__ bias,
                     const float* __restrict__ lower, int n_qf, int n_v, float* __restrict__ qf,
                     float* __restrict__ v) {
  pdl_wait_block();
  pdl_launch_dependents();
  // Grid (token, slice of 256 channels): one channel per thread, so that a step of a few tokens
  // is many short blocks rather than a few that loop.
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const T* x = pre + (size_t)t * row_width;
  float* out = qf + (size_t)t * 2 * n_qf;
  if (c < n_qf) {
    const float pq = to_f32<T>(x[c]);
    const float l = lower[c];
    out[c] = pq * sigmoid_f32(pq);
    out[n_qf + c] = l + (1.0f - l) * sigmoid_f32(to_f32<T>(x[n_qf + c]) + bias[c]);
  }
  if (c < n_v) v[(size_t)t * n_v + c] = to_f32<T>(x[2 * n_qf + c]);
}

template <int RS, int ROWS, bool VEC>
__global__ void __launch_bounds__(256)
forget_scan_kernel(const float* __restrict__ qf, const float* __restrict__ v, float* __restrict__ state,
                   const int* __restrict__ cu_q, const int* __restrict__ slots, int num_slots, int H, int d, int dv,
                   int cols, int nbuf, float* __restrict__ out, int* err) {
  pdl_wait_block();
  pdl_launch_dependents();
  // A ring of nbuf (2 or 4) buffers of: q [CHUNK][d], f [CHUNK][d], v [CHUNK][cols_pad].
  extern __shared__ __align__(16) float stage[];
  const int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * cols;
  const int rs = threadIdx.x % RS, col_local = threadIdx.x / RS;
  const int col = col0 + col_local;
  const bool on = col_local < cols && col < dv;
  const int first = cu_q[b], n = cu_q[b + 1] - first;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, SB_ERR_BAD_SLOT);
    return;
  }
  const int cols_pad = (cols + 3) & ~3;
  const int buffer = FORGET_CHUNK * (2 * d + cols_pad);
  const int n_qf = H * d;

  auto issue = [&](int which, int base) {
    float* buf = stage + which * buffer;
    const int count = min(FORGET_CHUNK, n - base);
    if (VEC) {
      const int d4 = d >> 2;
      for (int idx = threadIdx.x; idx < count * 2 * d4; idx += blockDim.x) {
        const int i = idx / (2 * d4), rem = idx - i * 2 * d4, kind = rem / d4, c = (rem - kind * d4) * 4;
        scan_copy16(buf + (kind * FORGET_CHUNK + i) * d + c,
                    qf + ((size_t)(first + base + i) * 2 + kind) * n_qf + h * d + c);
      }
    } else {
      for (int idx = threadIdx.x; idx < count * 2 * d; idx += blockDim.x) {
        const int i = idx / (2 * d), rem = idx - i * 2 * d, kind = rem / d, c = rem - kind * d;
        scan_copy4(buf + (kind * FORGET_CHUNK + i) * d + c,
                   qf + ((size_t)(first + base + i) * 2 + kind) * n_qf + h * d + c);
      }
    }
    float* bv = buf + 2 * FORGET_CHUNK * d;
    for (int idx = threadIdx.x; idx < count * cols; idx += blockDim.x) {
      const int i = idx / cols, c = idx - i * cols;
      scan_copy4(bv + i * cols_pad + c, v + ((size_t)(first + base + i) * H + h) * dv + min(col0 + c, dv - 1));
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  // The walk over a chunk is shorter than a chunk's way from memory (every column tile of a head
  // fetches the head's q and f): nbuf - 1 chunks are under way at any time.
  for (int p = 0; p < nbuf - 1; ++p) {
    if (p * FORGET_CHUNK < n) issue(p, p * FORGET_CHUNK);
    else asm volatile("cp.async.commit_group;\n" ::);
  }
  float* S = state + ((size_t)slot * H + h) * d * dv;
  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = VEC ? 4 * (rs + RS * (r >> 2)) + (r & 3) : rs + RS * r;
    s[r] = (on && row < d) ? S[(size_t)row * dv + col] : 0.f;
  }
  int which = 0;
  for (int base = 0; base < n; base += FORGET_CHUNK, which = which + 1 == nbuf ? 0 : which + 1) {
    const int count = min(FORGET_CHUNK, n - base);
    const int ahead = base + (nbuf - 1) * FORGET_CHUNK;  // goes where the chunk before this one was
    if (ahead < n) issue(which == 0 ? nbuf - 1 : which - 1, ahead);
    else asm volatile("cp.async.commit_group;\n" ::);
    if (nbuf == 4) asm volatile("cp.async.wait_group 3;\n" ::);
    else asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    const float* buf = stage + which * buffer;
    int i = 0;
    if constexpr (VEC) {
      // Several tokens at a time: a row's state goes through their updates in one chain of
      // multiply-adds, the sums that read it are chains of their own, and their sums over lanes go
      // side by side, so that a token's latencies are paid once per group of tokens.
      const float* vbuf = buf + 2 * FORGET_CHUNK * d + min(col_local, cols - 1);
      for (; i + FORGET_TOGETHER <= count; i += FORGET_TOGETHER) {
        float od4[FORGET_TOGETHER], vv4[FORGET_TOGETHER];
#pragma unroll
        for (int t = 0; t < FORGET_TOGETHER; ++t) {
          vv4[t] = vbuf[(i + t) * cols_pad];
          od4[t] = 0.f;
        }
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const int at = rs + RS * r;
          if (4 * at < d) {
#pragma unroll
            for (int t = 0; t < FORGET_TOGETHER; ++t) {
              const float4 f4 = reinterpret_cast<const float4*>(buf + (FORGET_CHUNK + i + t) * d)[at];
              const float4 q4 = reinterpret_cast<const float4*>(buf + (i + t) * d)[at];
              s[4 * r] = fmaf(f4.x, s[4 * r], (1.0f - f4.x) * vv4[t]);
              s[4 * r + 1] = fmaf(f4.y, s[4 * r + 1], (1.0f - f4.y) * vv4[t]);
              s[4 * r + 2] = fmaf(f4.z, s[4 * r + 2], (1.0f - f4.z) * vv4[t]);
              s[4 * r + 3] = fmaf(f4.w, s[4 * r + 3], (1.0f - f4.w) * vv4[t]);
              od4[t] = fmaf(s[4 * r], q4.x, od4[t]);
              od4[t] = fmaf(s[4 * r + 1], q4.y, od4[t]);
              od4[t] = fmaf(s[4 * r + 2], q4.z, od4[t]);
              od4[t] = fmaf(s[4 * r + 3], q4.w, od4[t]);
            }
          }
        }
#pragma unroll
        for (int o = 1; o < RS; o <<= 1) {
#pragma unroll
          for (int t = 0; t < FORGET_TOGETHER; ++t) od4[t] += __shfl_xor_sync(0xffffffffu, od4[t], o);
        }
        if (on && rs == 0) {
          float* dst = out + ((size_t)(first + base + i) * H + h) * dv + col;
#pragma unroll
          for (int t = 0; t < FORGET_TOGETHER; ++t) dst[(size_t)t * H * dv] = od4[t];
        }
      }
    }
    for (; i < count; ++i) {
      const float* qq = buf + i * d;
      const float* ff = buf + (FORGET_CHUNK + i) * d;
      const float vv = buf[2 * FORGET_CHUNK * d + i * cols_pad + min(col_local, cols - 1)];
      float od;
      if constexpr (VEC) {
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
        for (int r = 0; r < ROWS / 4; ++r) {
          const int at = rs + RS * r;
          if (4 * at < d) {
            const float4 f4 = reinterpret_cast<const float4*>(ff)[at];
            const float4 q4 = reinterpret_cast<const float4*>(qq)[at];
            s[4 * r] = fmaf(f4.x, s[4 * r], (1.0f - f4.x) * vv); o0 = fmaf(s[4 * r], q4.x, o0);
            s[4 * r + 1] = fmaf(f4.y, s[4 * r + 1], (1.0f - f4.y) * vv); o1 = fmaf(s[4 * r + 1], q4.y, o1);
            s[4 * r + 2] = fmaf(f4.z, s[4 * r + 2], (1.0f - f4.z) * vv); o2 = fmaf(s[4 * r + 2], q4.z, o2);
            s[4 * r + 3] = fmaf(f4.w, s[4 * r + 3], (1.0f - f4.w) * vv); o3 = fmaf(s[4 * r + 3], q4.w, o3);
          }
        }
        od = (o0 + o1) + (o2 + o3);
      } else {
        od = 0.f;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const int row = rs + RS * r;
          if (row < d) {
            const float f = ff[row];
            s[r] = fmaf(f, s[r], (1.0f - f) * vv);
            od = fmaf(s[r], qq[row], od);
          }
        }
      }
#pragma unroll
      for (int o = 1; o < RS; o <<= 1) od += __shfl_xor_sync(0xffffffffu, od, o);
      if (on && rs == 0) out[((size_t)(first + base + i) * H + h) * dv + col] = od;
    }
    __syncthreads();  // the buffer is filled again in the next round
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (on && first_row_of_slot(slots, b)) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = VEC ? 4 * (rs + RS * (r >> 2)) + (r & 3) : rs + RS * r;
      if (row < d) S[(size_t)row * dv + col] = s[r];
    }
  }
}

// scratch: float32 [T, 2 H d + H dv] for the inputs.
extern "C" int sb_forget_scan(const void* pre, int row_width, int dtype, const float* bias, const float* lower,
                              float* state, const int* cu_q, const int* slots, int num_tokens, int num_seqs,
                              int num_slots, int H, int d, int dv, int max_q_len, float* scratch, float* out,
                              int* err, cudaStream_t stream) {
  if (num_seqs == 0 || num_tokens == 0) return 0;
  if (d <= 0 || d > 32 * 32 || dv <= 0 || H <= 0) return -13;
  float* qf = scratch;
  float* v = scratch + (size_t)num_tokens * 2 * H * d;
  const int widest = H * d > H * dv ? H * d : H * dv;
  const dim3 in_grid((unsigned)num_tokens, (unsigned)((widest + 255) / 256));
  if (dtype == SB_DTYPE_F32)
    sb_launch(forget_inputs_kernel<float>, in_grid, 256, 0, stream, (const float*)pre, row_width, bias, lower,
              H * d, H * dv, qf, v);
  else
    sb_launch(forget_inputs_kernel<bf16>, in_grid, 256, 0, stream, (const bf16*)pre, row_width, bias, lower,
              H * d, H * dv, qf, v);
  SB_LAUNCH_CHECK();
  const bool vec = d % 4 == 0;
  const int rows = (vec && d <= 8 * 32) ? 8 : 32;
  int rs = 1;
  while (rs * rows < d) rs <<= 1;
  // Long walks: blocks of 128 threads (more blocks, each a chain of its own).  Steps of a few tokens
  // read and write the state and little else: 256 threads, so that a block's columns of a state row
  // are whole 32-byte sectors (16 columns of a row for heads of 128 channels).
  const int threads = max_q_len >= 64 ? 128 : 256;
  int cols = threads / rs;
  if (cols < 1) cols = 1;
  if (cols > dv) cols = dv;
  const int block = ((cols * rs + 31) / 32) * 32;
  const dim3 grid(H, num_seqs, (dv + cols - 1) / cols);
  const size_t one = (size_t)FORGET_CHUNK * (2 * d + ((cols + 3) & ~3)) * sizeof(float);
  const int nbuf = (max_q_len > 2 * FORGET_CHUNK && 4 * one <= 100 * 1024) ? 4 : 2;
  const size_t smem = nbuf * one;
  if (smem > 200 * 1024) return -13;
#define SB_FORGET_V(RS_, ROWS_, VEC_)                                                                          \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(forget_scan_kernel<RS_, ROWS_, VEC_>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                           (int)smem);                                                                         \
    if (max_q_len >= 64)                                                                                       \
      sb_launch_plain(forget_scan_kernel<RS_, ROWS_, VEC_>, grid, block, smem, stream, (const float*)qf,       \
                      (const float*)v, state, cu_q, slots, num_slots, H, d, dv, cols, nbuf, out, err);         \
    else                                                                                                       \
      sb_launch(forget_scan_kernel<RS_, ROWS_, VEC_>, grid, block, smem, stream, (const float*)qf,             \
                (const float*)v, state, cu_q, slots, num_slots, H, d, dv, cols, nbuf, out, err);               \
  } while (0)
#define SB_FORGET(RS_)                                \
  do {                                                \
    if (rows == 8) SB_FORGET_V(RS_, 8, true);         \
    else if (vec) SB_FORGET_V(RS_, 32, true);         \
    else SB_FORGET_V(RS_, 32, false);                 \
  } while (0)
  switch (rs) {
    case 1: SB_FORGET(1); break;
    case 2: SB_FORGET(2); break;
    case 4: SB_FORGET(4); break;
    case 8: SB_FORGET(8); break;
    case 16: SB_FORGET(16); break;
    default: SB_FORGET(32); break;
  }
#undef SB_FORGET
#undef SB_FORGET_V
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Output of a recurrent mixer: per head RMS norm, channel scale, and (gate_offset >= 0) a gate read
// from `low`.  One block per token, a warp per head.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
gated_head_norm_kernel(const float* __restrict__ o, const T* __restrict__ low, int low_width, int gate_offset,
                       const float* __restrict__ w, float eps, int H, int dv, T* __restrict__ out) {
  pdl_wait_block();
  pdl_launch_dependents();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int h = warp; h < H; h += nwarps) {
    const float* src = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) {
      const float gate = gate_offset < 0 ? 1.0f
          : sigmoid_f32(to_f32<T>(low[(size_t)t * low_width + gate_offset + h * dv + c]));
      out[((size_t)t * H + h) * dv + c] = from_f32<T>(src[c] * rstd * w[c] * gate);
    }
  }
}

extern "C" int sb_gated_head_norm(const float* o, const void* low, int low_width, int gate_offset, int dtype,
                                  const float* w, float eps, int num_tokens, int H, int dv, void* out,
                                  cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (dtype == SB_DTYPE_F32)
    sb_launch(gated_head_norm_kernel<float>, num_tokens, 256, 0, stream, o, (const float*)low, low_width,
              gate_offset, w, eps, H, dv, (float*)out);
  else
    sb_launch(gated_head_norm_kernel<bf16>, num_tokens, 256, 0, stream, o, (const bf16*)low, low_width,
              gate_offset, w, eps, H, dv, (bf16*)out);
  SB_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------
// Mean of up to four RMS-normed branches.  One block per token.
// ---------------------------------------------------------------------------
struct MeanBranches {
  const void* x[4];
  const float* w[4];
};

template <typename T>
__global__ void __launch_bounds__(256)
normed_mean_kernel(MeanBranches br, int count, float eps, int width, T* __restrict__ out) {
  pdl_wait_block();
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  constexpr int N = Vec<T>::N;
  const bool vec = width % N == 0;
  float rstd[4];
  for (int i = 0; i < count; ++i) {
    const T* x = reinterpret_cast<const T*>(br.x[i]) + (size_t)t * width;
    float ss = 0.f;
    if (vec) {
      for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {
        float a[N];
        Vec<T>::load(x + c, a);
#pragma unroll
        for (int e = 0; e < N; ++e) ss = fmaf(a[e], a[e], ss);
      }
    } else {
      for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float a = to_f32<T>(x[c]);
        ss = fmaf(a, a, ss);
      }
    }
    ss = block_sum(ss, scratch);
    rstd[i] = 1.0f / sqrtf(ss / (float)width + eps);
  }
  const float share = 1.0f / (float)count;
  if (vec) {
    for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {
      float acc[N];
#pragma unroll
      for (int e = 0; e < N; ++e) acc[e] = 0.f;
      for (int i = 0; i < count; ++i) {
        float a[N], w[N];
        Vec<T>::load(reinterpret_cast<const T*>(br.x[i]) + (size_t)t * width + c, a);
#pragma unroll
        for (int e = 0; e < N; e += 4) Vec<float>::load(br.w[i] + c + e, w + e);
#pragma unroll
        for (int e = 0; e < N; ++e) acc[e] += a[e] * rstd[i] * w[e];
      }
#pragma unroll
      for (int e = 0; e < N; ++e) acc[e] *= share;
      Vec<T>::store(out + (size_t)t * width + c, acc);
    }
    return;
  }
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < count; ++i)
      acc += to_f32<T>(reinterpret_cast<const T*>(br.x[i])[(size_t)t * width + c]) * rstd[i] * br.w[i][c];
    out[(size_t)t * width + c] = from_f32<T>(acc * share);
  }
}

extern "C" int sb_normed_mean(const void* x0, const void* x1, const void* x2, const void* x3, const float* w0,
                              const float* w1, const float* w2, const float* w3, int count, int dtype, float eps,
                              int num_tokens, int width, void* out, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (count < 1 || count > 4) return -13;
  MeanBranches br = {{x0, x1, x2, x3}, {w0, w1, w2, w3}};
  if (dtype == SB_DTYPE_F32)
    sb_launch(normed_mean_kernel<float>, num_tokens, 256, 0, stream, br, count, eps, width, (float*)out);
  else
    sb_launch(normed_mean_kernel<bf16>, num_tokens, 256, 0, stream, br, count, eps, width, (bf16*)out);
  SB_LAUNCH_CHECK();
  return 0;
}
