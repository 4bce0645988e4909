// Gated linear attention: linear attention whose state decays by a factor of its own per key channel and per token,
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t        (S is [dim, vdim] per (sequence, head)),
// with alpha_t = sigmoid(z_t)^(1/tau) from a projection z of the token.  Prompts (any number of tokens per sequence,
// continued from the state an earlier step left) and decoding (one token) run the same kernel.  Everything after the
// projections is 32-bit: q and k, the decay and its logarithm, the state, o.  The per-head norm and the gate that
// follow are retention's (retention_gate with a weight).
//
//   gla_prepare   q (times q_scale), k of the projection's row as float, and alpha = exp(log sigmoid(z) / tau) with
//                 log sigmoid(z) = min(z, 0) - log1p(exp(-|z|)): float [3, T, heads*dim]
//   gla_scan      the recurrence, token by token.  The state of a (sequence, head) is kept as [vdim][dim] (a column of
//                 S, one value dimension, is contiguous), like retention's.  A block owns (sequence, head, a slice of
//                 value columns); the columns of S are independent of each other, so the slices never talk.  A warp
//                 owns CPW columns and a lane the rows lane, lane + 32, ... of each in registers, so one load of a
//                 token's q, k and alpha from shared memory serves CPW columns.  The order of every sum is fixed by
//                 (dim, position in the sequence) alone: how a prompt is cut into steps, what else is in the batch
//                 and how many columns a warp holds change no bit.
#include "common.cuh"

#define GL_WARPS 8            // warps of a scan block
#define GL_TOK 16             // tokens staged in shared memory at a time

template <typename T>
__global__ void gla_prepare_kernel(const T* __restrict__ src, int row_stride, int q_col, int k_col,
                                   const float* __restrict__ z, float* __restrict__ qka, int width, float q_scale,
                                   float inv_tau, int T_) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)T_ * width;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width, c = idx - t * width;
        qka[idx] = Cvt<T>::to_f32(src[t * row_stride + q_col + c]) * q_scale;
        qka[n + idx] = Cvt<T>::to_f32(src[t * row_stride + k_col + c]);
        const float zz = z[idx];
        const float log_sig = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
        qka[2 * n + idx] = expf(log_sig * inv_tau);
    }
}

// grid (sequence, head, ceil(vdim / (GL_WARPS * CPW))); R = ceil(dim / 32) rows of a column per lane.
template <typename T, int R, int CPW>
__global__ void __launch_bounds__(GL_WARPS * 32)
gla_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ alpha,
                const T* __restrict__ v, int v_stride, float* __restrict__ state, float* __restrict__ o,
                const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
    constexpr int COLS = GL_WARPS * CPW;
    extern __shared__ float sh[];                     // q, k, alpha [GL_TOK][dim] each, v [GL_TOK][COLS]
    float* qs = sh;
    float* ks = qs + GL_TOK * dim;
    float* as = ks + GL_TOK * dim;
    float* vs = as + GL_TOK * dim;
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = cu_q[b], row1 = cu_q[b + 1];
    const int slot = seq_slot[b];
    const int width = heads * dim;
    float* S = state + ((size_t)slot * heads + h) * vdim * dim;
    pdl_wait();
    float s[CPW][R];
#pragma unroll
    for (int c = 0; c < CPW; ++c) {
        const int j = j0 + warp * CPW + c;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = lane + 32 * r;
            s[c][r] = (i < dim && j < vdim) ? S[(size_t)j * dim + i] : 0.f;
        }
    }
    for (int t0 = row0; t0 < row1; t0 += GL_TOK) {
        const int cnt = min(GL_TOK, row1 - t0);
        __syncthreads();                              // the tokens before are used up
        for (int idx = threadIdx.x; idx < cnt * dim; idx += blockDim.x) {
            const int tt = idx / dim, i = idx - tt * dim;
            const size_t g = (size_t)(t0 + tt) * width + h * dim + i;
            qs[idx] = q[g];
            ks[idx] = k[g];
            as[idx] = alpha[g];
        }
        for (int idx = threadIdx.x; idx < cnt * COLS; idx += blockDim.x) {
            const int tt = idx / COLS, c = idx - tt * COLS;
            vs[idx] = (j0 + c < vdim) ? Cvt<T>::to_f32(v[(size_t)(t0 + tt) * v_stride + h * vdim + j0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 2
        for (int tt = 0; tt < cnt; ++tt) {
            float vj[CPW], acc[CPW];
#pragma unroll
            for (int c = 0; c < CPW; ++c) { vj[c] = vs[tt * COLS + warp * CPW + c]; acc[c] = 0.f; }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = lane + 32 * r;
                if (i < dim) {
                    const float a = as[tt * dim + i], kk = ks[tt * dim + i], qq = qs[tt * dim + i];
#pragma unroll
                    for (int c = 0; c < CPW; ++c) {
                        s[c][r] = fmaf(a, s[c][r], kk * vj[c]);
                        acc[c] = fmaf(s[c][r], qq, acc[c]);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < CPW; ++c) {
                const float sum = warp_sum(acc[c]);
                const int j = j0 + warp * CPW + c;
                if (lane == 0 && j < vdim) o[(size_t)(t0 + tt) * heads * vdim + h * vdim + j] = sum;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < CPW; ++c) {
        const int j = j0 + warp * CPW + c;
        if (j < vdim) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = lane + 32 * r;
                if (i < dim) S[(size_t)j * dim + i] = s[c][r];
            }
        }
    }
}

template <typename T, int R, int CPW>
static int launch_scan_rc(const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                          float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim,
                          cudaStream_t st) {
    constexpr int COLS = GL_WARPS * CPW;
    const size_t smem = (size_t)(3 * GL_TOK * dim + GL_TOK * COLS) * sizeof(float);
    const int gz = (vdim + COLS - 1) / COLS;
    if (gz > 65535) return RF_ERR_UNSUPPORTED;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<T, R, CPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    rf_launch(gla_scan_kernel<T, R, CPW>, dim3(B, heads, gz), dim3(GL_WARPS * 32), smem, st, q, k, alpha,
              reinterpret_cast<const T*>(v), v_stride, state, o, cu_q, seq_slot, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T, int R>
static int launch_scan_r(const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                         float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, int sms,
                         cudaStream_t st) {
    // columns per warp: as many as still leave about two blocks per SM (a column's arithmetic is the same in all three)
    const long long groups = (long long)B * heads;
    if (R <= 4 && groups * ((vdim + 8 * 4 - 1) / (8 * 4)) >= 2LL * sms)
        return launch_scan_rc<T, R, 4>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, st);
    if (groups * ((vdim + 8 * 2 - 1) / (8 * 2)) >= 2LL * sms)
        return launch_scan_rc<T, R, 2>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, st);
    return launch_scan_rc<T, R, 1>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, st);
}

template <typename T>
static int launch_scan(const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                       float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, int sms,
                       cudaStream_t st) {
    if (B <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || heads <= 0 || heads > 65535) return RF_ERR_UNSUPPORTED;
    if (sms <= 0) sms = 148;
#define GL_CASE(R) return launch_scan_r<T, R>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, sms, st)
    switch ((dim + 31) / 32) {
        case 1: GL_CASE(1);
        case 2: GL_CASE(2);
        case 3: GL_CASE(3);
        case 4: GL_CASE(4);
        case 5: case 6: GL_CASE(6);
        default: GL_CASE(8);
    }
#undef GL_CASE
}

template <typename T>
static int launch_prepare(const void* src, int row_stride, int q_col, int k_col, const float* z, float* qka, int width,
                          float q_scale, float tau, int T_, cudaStream_t st) {
    const size_t n = (size_t)T_ * width;
    if (n == 0) return 0;
    if (!(tau > 0.f)) return RF_ERR_BAD_ARG;
    const size_t blocks = (n + 255) / 256;
    rf_launch(gla_prepare_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st,
              reinterpret_cast<const T*>(src), row_stride, q_col, k_col, z, qka, width, q_scale, 1.f / tau, T_);
    RF_LAUNCH_CHECK();
    return 0;
}

// dtype: 0 = float32, 1 = bfloat16 (of the projection's output and of v)
extern "C" {
// src [T, row_stride]: q at columns q_col.., k at k_col.. (width = heads*dim each); z float [T, width]; qka float [3, T, width]
int rf_gla_prepare(int dtype, const void* src, int row_stride, int q_col, int k_col, const float* z, float* qka, int width,
                   float q_scale, float tau, int T_, cudaStream_t st) {
    return dtype == 0 ? launch_prepare<float>(src, row_stride, q_col, k_col, z, qka, width, q_scale, tau, T_, st)
                      : launch_prepare<__nv_bfloat16>(src, row_stride, q_col, k_col, z, qka, width, q_scale, tau, T_, st);
}
// state float [slots, heads, vdim, dim]; o float [T, heads*vdim]; sms: multiprocessors of the device (sizes the blocks)
int rf_gla_scan(int dtype, const float* q, const float* k, const float* alpha, const void* v, int v_stride, float* state,
                float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, int sms, cudaStream_t st) {
    return dtype == 0 ? launch_scan<float>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, sms, st)
                      : launch_scan<__nv_bfloat16>(q, k, alpha, v, v_stride, state, o, cu_q, seq_slot, B, heads, dim, vdim, sms, st);
}
}
