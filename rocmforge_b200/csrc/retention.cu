// Retention: linear attention with a fixed decay per head and a matrix state per (sequence, head),
//   S_t = decay_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,
// for prompts (any number of tokens per sequence, continued from the state an earlier step left) and for
// decoding (one token), by the same kernels.  Everything after the projections is 32-bit: the rotation's angle,
// q and k after rotation, the state, o, its per-head unit norm.
//
//   retention_prepare   q, k of the projection's row -> rotated (first rot_dim elements of a head, pairs
//                       (i, i + rot_dim/2), angle float(pos) * inv_freq[i]), k scaled, as float [2, T, heads*dim]
//   retention_scan      the recurrence, token by token: a block owns (sequence, head, a slice of 8 value columns);
//                       the columns of S are independent of each other, so the slices never talk.  A warp owns one
//                       column; a lane holds the rows lane, lane + 32, ... of it in registers.  The order of every sum
//                       is fixed by (dim, position in the sequence) alone: how a prompt is cut into steps, or what
//                       else is in the batch, changes no bit.
//   retention_gate      o / rms(o) per head, times silu(gate), into the compute dtype for the output product
#include "common.cuh"

#define RT_COLS 8             // value columns (warps) of a scan block
#define RT_TOK 16             // tokens staged in shared memory at a time

template <typename T>
__global__ void retention_prepare_kernel(const T* __restrict__ src, int row_stride, int q_col, int k_col,
                                         float* __restrict__ qk, int heads, int dim, int rot_dim,
                                         const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                                         float k_scale, int T_) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int width = heads * dim;
    const int pos = tok_pos[t];
    const int rh = rot_dim >> 1;
    pdl_wait();
    for (int idx = threadIdx.x; idx < 2 * width; idx += blockDim.x) {
        const int which = idx >= width;                       // 0: q, 1: k
        const int c = idx - which * width, e = c % dim;
        const T* row = src + (size_t)t * row_stride + (which ? k_col : q_col);
        float x = Cvt<T>::to_f32(row[c]);
        if (e < rot_dim) {
            const bool first = e < rh;
            const int i = first ? e : e - rh;
            const float y = Cvt<T>::to_f32(row[first ? c + rh : c - rh]);
            float s, cs;
            sincosf((float)pos * inv_freq[i], &s, &cs);
            x = first ? x * cs - y * s : x * cs + y * s;
        }
        if (which) x *= k_scale;
        qk[(size_t)which * T_ * width + (size_t)t * width + c] = x;
    }
}

// grid (sequence, head, ceil(vdim / RT_COLS)); block RT_COLS warps.  R = ceil(dim / 32) rows of a column per lane.
template <typename T, int R>
__global__ void __launch_bounds__(RT_COLS * 32)
retention_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const T* __restrict__ v, int v_stride,
                      float* __restrict__ state, const float* __restrict__ decay, float* __restrict__ o,
                      const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int heads, int dim, int vdim) {
    extern __shared__ float sh[];                     // q [RT_TOK][dim], k [RT_TOK][dim], v [RT_TOK][RT_COLS]
    float* qs = sh;
    float* ks = qs + RT_TOK * dim;
    float* vs = ks + RT_TOK * dim;
    pdl_trigger();
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * RT_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = j0 + warp;
    const int row0 = cu_q[b], row1 = cu_q[b + 1];
    const int slot = seq_slot[b];
    const float d = decay[h];
    const int width = heads * dim;
    float* S = state + (((size_t)slot * heads + h) * dim) * vdim;
    pdl_wait();
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = lane + 32 * r;
        s[r] = (i < dim && j < vdim) ? S[(size_t)i * vdim + j] : 0.f;
    }
    for (int t0 = row0; t0 < row1; t0 += RT_TOK) {
        const int cnt = min(RT_TOK, row1 - t0);
        __syncthreads();                              // the tokens before are used up
        for (int idx = threadIdx.x; idx < cnt * dim; idx += blockDim.x) {
            const int tt = idx / dim, i = idx - tt * dim;
            qs[idx] = q[(size_t)(t0 + tt) * width + h * dim + i];
            ks[idx] = k[(size_t)(t0 + tt) * width + h * dim + i];
        }
        for (int idx = threadIdx.x; idx < cnt * RT_COLS; idx += blockDim.x) {
            const int tt = idx / RT_COLS, c = idx - tt * RT_COLS;
            vs[idx] = (j0 + c < vdim) ? Cvt<T>::to_f32(v[(size_t)(t0 + tt) * v_stride + h * vdim + j0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 4
        for (int tt = 0; tt < cnt; ++tt) {
            const float vj = vs[tt * RT_COLS + warp];
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = lane + 32 * r;
                if (i < dim) {
                    s[r] = fmaf(d, s[r], ks[tt * dim + i] * vj);
                    acc = fmaf(s[r], qs[tt * dim + i], acc);
                }
            }
            acc = warp_sum(acc);
            if (lane == 0 && j < vdim) o[(size_t)(t0 + tt) * heads * vdim + h * vdim + j] = acc;
        }
    }
    if (j < vdim) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = lane + 32 * r;
            if (i < dim) S[(size_t)i * vdim + j] = s[r];
        }
    }
}

// a warp per (token, head): out = o / sqrt(mean(o^2) + eps) * silu(gate)
template <typename T>
__global__ void retention_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                                      T* __restrict__ out, int heads, int vdim, float eps, int T_) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long total = (long long)T_ * heads;
    for (long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < total;
         w += (long long)gridDim.x * (blockDim.x >> 5)) {
        const long long t = w / heads;
        const int h = (int)(w - t * heads);
        const float* orow = o + (size_t)t * heads * vdim + (size_t)h * vdim;
        float ss = 0.f;
        for (int e = lane; e < vdim; e += 32) ss += orow[e] * orow[e];
        const float r = rsqrtf(warp_sum(ss) / (float)vdim + eps);
        for (int e = lane; e < vdim; e += 32) {
            const float g = Cvt<T>::to_f32(gate[(size_t)t * gate_stride + (size_t)h * vdim + e]);
            out[(size_t)t * heads * vdim + (size_t)h * vdim + e] = Cvt<T>::from_f32(orow[e] * r * (g / (1.f + expf(-g))));
        }
    }
}

template <typename T>
static int launch_prepare(const void* src, int row_stride, int q_col, int k_col, float* qk, int heads, int dim,
                          int rot_dim, const float* inv_freq, const int* tok_pos, float k_scale, int T_, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (rot_dim < 0 || rot_dim % 2 || rot_dim > dim) return RF_ERR_BAD_ARG;
    rf_launch(retention_prepare_kernel<T>, dim3(T_), dim3(256), 0, st, reinterpret_cast<const T*>(src), row_stride, q_col, k_col,
              qk, heads, dim, rot_dim, inv_freq, tok_pos, k_scale, T_);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T, int R>
static int launch_scan_r(const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                         float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, cudaStream_t st) {
    const size_t smem = (size_t)(2 * RT_TOK * dim + RT_TOK * RT_COLS) * sizeof(float);
    dim3 grid(B, heads, (vdim + RT_COLS - 1) / RT_COLS);
    rf_launch(retention_scan_kernel<T, R>, grid, dim3(RT_COLS * 32), smem, st, q, k, reinterpret_cast<const T*>(v), v_stride, state,
              decay, o, cu_q, seq_slot, heads, dim, vdim);
    RF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_scan(const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                       float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, cudaStream_t st) {
    if (B <= 0) return 0;
    if (dim <= 0 || dim > 256 || vdim <= 0 || heads <= 0 || heads > 65535 || (vdim + RT_COLS - 1) / RT_COLS > 65535)
        return RF_ERR_UNSUPPORTED;
    switch ((dim + 31) / 32) {
        case 1: return launch_scan_r<T, 1>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 2: return launch_scan_r<T, 2>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 3: return launch_scan_r<T, 3>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 4: return launch_scan_r<T, 4>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        case 5: case 6: return launch_scan_r<T, 6>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
        default: return launch_scan_r<T, 8>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
    }
}

template <typename T>
static int launch_gate(const float* o, const void* gate, int gate_stride, void* out, int heads, int vdim, float eps, int T_,
                       cudaStream_t st) {
    const long long total = (long long)T_ * heads;
    if (total <= 0) return 0;
    const long long blocks = (total + 7) / 8;
    rf_launch(retention_gate_kernel<T>, dim3((unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks)), dim3(256), 0, st, o,
              reinterpret_cast<const T*>(gate), gate_stride, reinterpret_cast<T*>(out), heads, vdim, eps, T_);
    RF_LAUNCH_CHECK();
    return 0;
}

// dtype: 0 = float32, 1 = bfloat16 (of the projection's output, of v, of the gate and of the gated result)
extern "C" {
int rf_retention_prepare(int dtype, const void* src, int row_stride, int q_col, int k_col, float* qk, int heads, int dim,
                         int rot_dim, const float* inv_freq, const int* tok_pos, float k_scale, int T_, cudaStream_t st) {
    return dtype == 0 ? launch_prepare<float>(src, row_stride, q_col, k_col, qk, heads, dim, rot_dim, inv_freq, tok_pos, k_scale, T_, st)
                      : launch_prepare<__nv_bfloat16>(src, row_stride, q_col, k_col, qk, heads, dim, rot_dim, inv_freq, tok_pos, k_scale, T_, st);
}
int rf_retention_scan(int dtype, const float* q, const float* k, const void* v, int v_stride, float* state, const float* decay,
                      float* o, const int* cu_q, const int* seq_slot, int B, int heads, int dim, int vdim, cudaStream_t st) {
    return dtype == 0 ? launch_scan<float>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st)
                      : launch_scan<__nv_bfloat16>(q, k, v, v_stride, state, decay, o, cu_q, seq_slot, B, heads, dim, vdim, st);
}
int rf_retention_gate(int dtype, const float* o, const void* gate, int gate_stride, void* out, int heads, int vdim, float eps,
                      int T_, cudaStream_t st) {
    return dtype == 0 ? launch_gate<float>(o, gate, gate_stride, out, heads, vdim, eps, T_, st)
                      : launch_gate<__nv_bfloat16>(o, gate, gate_stride, out, heads, vdim, eps, T_, st);
}
}
