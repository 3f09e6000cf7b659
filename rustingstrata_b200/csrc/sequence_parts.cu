// Kernels of parts that carry a fixed-size state per request, and of blocks that norm a sublayer's output before it
// joins the residual stream:
//   * rmsnorm_add: x += norm(delta) (gain one number or a vector), optionally followed by out = norm2(x) for the next
//     reader of the stream, in one pass over the row;
//   * concat_embed: [x | table[id]] per token for a stream that re-reads the embedding, the stream then preset to a
//     row vector so that an accumulating product lands on it;
//   * short_conv: causal convolution over time on each channel for a packed batch of sequences cut anywhere, the last
//     taps - 1 inputs of every sequence kept in its state slot;
//   * block_linear: a block-diagonal matrix product (one small matrix per block of channels, strided in and out);
//   * gated_linear_recurrence: S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-c r_t softplus(lam)),
//     r and i sigmoids of given pre-activations, the output multiplied by a GELU branch; S lives in the state slot;
//   * latent_kv_write: latent norm, interleaved rotation, write of [latent | rotated key part] into a one-plane
//     cache page, rotation of the queries' rotated parts;
//   * activation: relu(x)^2.
// Norms, gates, decays, the recurrence and the rotation are float32 whatever the activation type is.  Every kernel
// computes a row (or a channel of a sequence) in an order that its own position fixes, never the batch.
#include "common.cuh"
#include <math.h>

namespace {
__device__ __forceinline__ void store_any(void* p, int dt, size_t i, float v) {
    if (dt == RS_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f32(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
}  // namespace

// --------------------------------------------------------------------------- norm of a sublayer's output into the stream
// x[r, :] += delta[r, :] * rsqrt(mean(delta[r]^2) + eps) * g      (g: one number when g_n == 1, else [n])
// and, when out != null: out[r, :] = x[r, :] * rsqrt(mean(x[r]^2) + eps2) * w2   (w2 likewise).
// A thread owns the same columns in every pass, so it re-reads what it wrote itself.
__global__ void rmsnorm_add_kernel(float* __restrict__ x, long x_stride, const float* __restrict__ delta, long d_stride,
                                   const void* __restrict__ g, int g_dt, int g_n, float eps,
                                   const void* __restrict__ w2, int w2_dt, int w2_n, float eps2,
                                   void* __restrict__ out, int out_dt, long out_stride, int n) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * x_stride;
    const float* dr = delta + (size_t)r * d_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float v = dr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float s = 1.0f / sqrtf(ss / (float)n + eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i] + dr[i] * s * load_any(g, g_dt, g_n == 1 ? 0 : i);
        xr[i] = v;
        ss2 = fmaf(v, v, ss2);
    }
    if (out == nullptr) return;
    ss2 = block_sum(ss2, scratch);
    const float s2 = 1.0f / sqrtf(ss2 / (float)n + eps2);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        store_any(out, out_dt, (size_t)r * out_stride + i, xr[i] * s2 * load_any(w2, w2_dt, w2_n == 1 ? 0 : i));
}

RS_EXPORT int rs_rmsnorm_add(float* x, long x_stride, const float* delta, long d_stride, const void* g, int g_dt, int g_n,
                             float eps, const void* w2, int w2_dt, int w2_n, float eps2, void* out, int out_dt,
                             long out_stride, int n_rows, int n, void* stream) {
    if (n_rows <= 0) return 0;
    const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
    rmsnorm_add_kernel<<<n_rows, threads, 0, (cudaStream_t)stream>>>(x, x_stride, delta, d_stride, g, g_dt, g_n, eps, w2,
                                                                     w2_dt, w2_n, eps2, out, out_dt, out_stride, n);
    return rs_launch_result();
}

// --------------------------------------------------------------------------- [x | embedding] and the stream preset
// cat[t, 0:n] = x[t, :] (rounded to the activation type), cat[t, n:2n] = table[ids[t], :]; then x[t, :] = row[:].
__global__ void concat_embed_kernel(float* __restrict__ x, long x_stride, const void* __restrict__ table, int table_dt,
                                    const int* __restrict__ ids, int V, const void* __restrict__ row, int row_dt,
                                    void* __restrict__ cat, int cat_dt, long cat_stride, int n, int* status) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(status, RS_STATUS_BAD_TOKEN);
        id = 0;
    }
    float* xr = x + (size_t)t * x_stride;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        store_any(cat, cat_dt, (size_t)t * cat_stride + i, xr[i]);
        store_any(cat, cat_dt, (size_t)t * cat_stride + n + i, load_any(table, table_dt, (size_t)id * n + i));
        xr[i] = row != nullptr ? load_any(row, row_dt, i) : 0.f;
    }
}

RS_EXPORT int rs_concat_embed(float* x, long x_stride, const void* table, int table_dt, const int* ids, int V,
                              const void* row, int row_dt, void* cat, int cat_dt, long cat_stride, int n_tokens, int n,
                              int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    concat_embed_kernel<<<n_tokens, 256, 0, (cudaStream_t)stream>>>(x, x_stride, table, table_dt, ids, V, row, row_dt, cat,
                                                                   cat_dt, cat_stride, n, status);
    return rs_launch_result();
}

// --------------------------------------------------------------------------- short causal convolution with state
// in: [T, C] (+ in_bias[c] on every real input).  For token row t of sequence s at local index li = t - q_start[s]:
//   out[t, c] = (add_input ? in(li) : 0) + bias[c] + sum_j w[c, j] * in(li - (taps - 1) + j),
// in(i) for i < 0 is the sequence's state tail[taps - 1 + i] (zero after admission: nothing before the start).
// tail: state[slot * state_stride + k * C + c], k = 0 the oldest.  w: [taps][C] (tap-major, so that neighbouring
// channels' weights of a tap are neighbours).
struct ConvParams {
    const void* in; int in_dt; long in_stride;
    const void* in_bias; int in_bias_dt;
    const void* w; int w_dt;
    const void* bias; int bias_dt;
    void* out; int out_dt; long out_stride;
    float* state; long state_stride;
    const int* seq_of_token; const int* q_start; const int* slots;
    int C, taps, add_input, n_tokens, n_seqs;
};

__device__ __forceinline__ float conv_input(const ConvParams& p, int row0, int i, int c, const float* tail) {
    if (i >= 0) {
        float v = load_any(p.in, p.in_dt, (size_t)(row0 + i) * p.in_stride + c);
        if (p.in_bias != nullptr) v += load_any(p.in_bias, p.in_bias_dt, c);
        return v;
    }
    return tail[(size_t)(p.taps - 1 + i) * p.C + c];
}

__global__ void short_conv_kernel(const ConvParams p) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)p.n_tokens * p.C) return;
    const int t = (int)(idx / p.C), c = (int)(idx % p.C);
    const int s = p.seq_of_token[t];
    const int row0 = p.q_start[s];
    const int li = t - row0;
    const float* tail = p.state + (size_t)p.slots[s] * p.state_stride;
    float acc = 0.f;
    for (int j = 0; j < p.taps; ++j)
        acc = fmaf(load_any(p.w, p.w_dt, (size_t)j * p.C + c), conv_input(p, row0, li - (p.taps - 1) + j, c, tail), acc);
    if (p.bias != nullptr) acc += load_any(p.bias, p.bias_dt, c);
    if (p.add_input) acc += conv_input(p, row0, li, c, tail);
    store_any(p.out, p.out_dt, (size_t)t * p.out_stride + c, acc);
}

// eight neighbouring channels per thread with 16- or 32-byte accesses (C and the row pitches multiples of 8, aligned)
__device__ __forceinline__ void load8(const void* p, int dt, size_t i, float* v) {
    if (dt == RS_F32) {
        const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
        const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int q = 0; q < 4; ++q) { v[2 * q] = __low2float(h[q]); v[2 * q + 1] = __high2float(h[q]); }
    }
}

__global__ void short_conv_vec_kernel(const ConvParams p) {
    const int groups = p.C >> 3;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)p.n_tokens * groups) return;
    const int t = (int)(idx / groups), c = (int)(idx % groups) << 3;
    const int s = p.seq_of_token[t];
    const int row0 = p.q_start[s];
    const int li = t - row0;
    const float* tail = p.state + (size_t)p.slots[s] * p.state_stride;
    float acc[8], x[8], w[8], ib[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { acc[e] = 0.f; ib[e] = 0.f; }
    if (p.in_bias != nullptr) load8(p.in_bias, p.in_bias_dt, c, ib);
    for (int j = 0; j < p.taps; ++j) {
        const int i = li - (p.taps - 1) + j;
        if (i >= 0) {
            load8(p.in, p.in_dt, (size_t)(row0 + i) * p.in_stride + c, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] += ib[e];
        } else {
            load8(tail, RS_F32, (size_t)(p.taps - 1 + i) * p.C + c, x);
        }
        load8(p.w, p.w_dt, (size_t)j * p.C + c, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(w[e], x[e], acc[e]);
    }
    if (p.bias != nullptr) {
        load8(p.bias, p.bias_dt, c, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += w[e];
    }
    if (p.add_input) {                                        // x still holds the current token's inputs (the last tap)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += x[e];
    }
    const size_t o = (size_t)t * p.out_stride + c;
    if (p.out_dt == RS_F32) {
        float* dst = reinterpret_cast<float*>(p.out) + o;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
        uint4 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = u;
    }
}

// the new tail: the last taps - 1 inputs of the sequence, old tail entries moving up when the step brought fewer
__global__ void short_conv_state_kernel(const ConvParams p) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)p.n_seqs * p.C) return;
    const int s = (int)(idx / p.C), c = (int)(idx % p.C);
    const int row0 = p.q_start[s], n = p.q_start[s + 1] - row0;
    float* tail = p.state + (size_t)p.slots[s] * p.state_stride;
    const int keep = p.taps - 1;
    float v[16];                                              // taps <= 17, checked by the launcher
    for (int k = 0; k < keep; ++k) v[k] = conv_input(p, row0, n - keep + k, c, tail);
    for (int k = 0; k < keep; ++k) tail[(size_t)k * p.C + c] = v[k];
}

// a step of single tokens: one thread per (sequence, channel) computes the output and moves the tail up, one kernel
__global__ void short_conv_single_kernel(const ConvParams p) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)p.n_seqs * p.C) return;
    const int s = (int)(idx / p.C), c = (int)(idx % p.C);
    const int row0 = p.q_start[s];
    float* tail = p.state + (size_t)p.slots[s] * p.state_stride;
    const float x = conv_input(p, row0, 0, c, tail);
    float acc = load_any(p.w, p.w_dt, (size_t)(p.taps - 1) * p.C + c) * x;
    for (int j = 0; j < p.taps - 1; ++j) {
        const float v = tail[(size_t)j * p.C + c];
        acc = fmaf(load_any(p.w, p.w_dt, (size_t)j * p.C + c), v, acc);
        if (j > 0) tail[(size_t)(j - 1) * p.C + c] = v;
    }
    if (p.taps > 1) tail[(size_t)(p.taps - 2) * p.C + c] = x;
    if (p.bias != nullptr) acc += load_any(p.bias, p.bias_dt, c);
    if (p.add_input) acc += x;
    store_any(p.out, p.out_dt, (size_t)row0 * p.out_stride + c, acc);
}

RS_EXPORT int rs_short_conv(const void* in, int in_dt, long in_stride, const void* in_bias, int in_bias_dt, const void* w,
                            int w_dt, const void* bias, int bias_dt, void* out, int out_dt, long out_stride, float* state,
                            long state_stride, const int* seq_of_token, const int* q_start, const int* slots, int C,
                            int taps, int add_input, int n_tokens, int n_seqs, void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (taps < 1 || taps > 17 || C <= 0) return (int)cudaErrorInvalidValue;
    ConvParams p{in, in_dt, in_stride, in_bias, in_bias_dt, w, w_dt, bias, bias_dt, out, out_dt, out_stride, state,
                 state_stride, seq_of_token, q_start, slots, C, taps, add_input, n_tokens, n_seqs};
    cudaStream_t s = (cudaStream_t)stream;
    if (n_tokens == n_seqs) {                     // every sequence brings one token
        const long st = (long)n_seqs * C;
        short_conv_single_kernel<<<(unsigned)((st + 255) / 256), 256, 0, s>>>(p);
        return rs_launch_result();
    }
    const long total = (long)n_tokens * C;
    auto aligned = [](const void* q, int dt) { return q == nullptr || ((size_t)q & (dt == RS_F32 ? 31 : 15)) == 0; };
    const bool vec = C % 8 == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 && state_stride % 8 == 0 && aligned(in, in_dt) &&
                     aligned(out, out_dt) && aligned(w, w_dt) && aligned(bias, bias_dt) && aligned(in_bias, in_bias_dt) &&
                     aligned(state, RS_F32);
    if (vec) short_conv_vec_kernel<<<(unsigned)((total / 8 + 255) / 256), 256, 0, s>>>(p);
    else short_conv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || taps == 1) return (int)e;
    const long st = (long)n_seqs * C;
    short_conv_state_kernel<<<(unsigned)((st + 255) / 256), 256, 0, s>>>(p);
    return rs_launch_result();
}

// --------------------------------------------------------------------------- block-diagonal matrix product
// out[t, b * out_bs + o] = bias[b * O + o] + sum_i W[b, o, i] * in[t, b * in_bs + i],  o < O, i < I, b < B.
// W: [B, O, I] contiguous.  Tiles of 64 x 64 outputs, k ascending per output element.
namespace {
constexpr int BL_BM = 64, BL_BN = 64, BL_BK = 16;

struct BlockLinearParams {
    const void* in; int in_dt; long in_stride; long in_bs;
    const void* w; int w_dt;
    const void* bias; int bias_dt;
    void* out; int out_dt; long out_stride; long out_bs;
    int T, O, I;
};

__global__ void __launch_bounds__(256) block_linear_kernel(const BlockLinearParams p) {
    __shared__ float As[BL_BK][BL_BM + 1];
    __shared__ float Ws[BL_BK][BL_BN + 1];
    const int tid = threadIdx.x, b = blockIdx.z;
    const int m0 = blockIdx.y * BL_BM, n0 = blockIdx.x * BL_BN;
    const int tx = tid % 16, ty = tid / 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const size_t w_base = (size_t)b * p.O * p.I;
    for (int k0 = 0; k0 < p.I; k0 += BL_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BL_BK, kk = idx % BL_BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < p.T && gk < p.I) ? load_any(p.in, p.in_dt, (size_t)gm * p.in_stride + (size_t)b * p.in_bs + gk) : 0.f;
            Ws[kk][r] = (gn < p.O && gk < p.I) ? load_any(p.w, p.w_dt, w_base + (size_t)gn * p.I + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BL_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= p.T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= p.O) continue;
            float v = acc[i][j];
            if (p.bias != nullptr) v += load_any(p.bias, p.bias_dt, (size_t)b * p.O + gn);
            store_any(p.out, p.out_dt, (size_t)gm * p.out_stride + (size_t)b * p.out_bs + gn, v);
        }
    }
}

// the same for at most 8 rows (single tokens): the rows sit in shared memory as float32, a warp owns output columns
// and reads their weight rows once, 16 bytes per lane and load where the weights are bfloat16 and aligned
constexpr int BR_ROWS = 8, BR_COLS = 32, BR_KC = 512;

__global__ void __launch_bounds__(256) block_linear_rows_kernel(const BlockLinearParams p) {
    __shared__ float xs[BR_ROWS][BR_KC];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, b = blockIdx.y;
    const int o0 = blockIdx.x * BR_COLS + warp * (BR_COLS / 8);
    float acc[BR_COLS / 8][BR_ROWS];
#pragma unroll
    for (int c = 0; c < BR_COLS / 8; ++c)
#pragma unroll
        for (int r = 0; r < BR_ROWS; ++r) acc[c][r] = 0.f;
    const bool vec = p.w_dt == RS_BF16 && p.I % 8 == 0 && ((size_t)p.w & 15) == 0;
    for (int k0 = 0; k0 < p.I; k0 += BR_KC) {
        __syncthreads();
        const int kc = min(BR_KC, p.I - k0);
        for (int i = tid; i < BR_ROWS * kc; i += 256) {
            const int r = i / kc, kk = i - r * kc;
            xs[r][kk] = r < p.T ? load_any(p.in, p.in_dt, (size_t)r * p.in_stride + (size_t)b * p.in_bs + k0 + kk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < BR_COLS / 8; ++c) {
            const int o = o0 + c;
            if (o >= p.O) continue;
            const size_t wrow = ((size_t)b * p.O + o) * p.I + k0;
            if (vec) {
                const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(p.w);
                for (int kk = lane * 8; kk < kc; kk += 256) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(wp + wrow + kk);
                    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float w0 = __low2float(w2[q]), w1 = __high2float(w2[q]);
#pragma unroll
                        for (int r = 0; r < BR_ROWS; ++r) acc[c][r] = fmaf(xs[r][kk + 2 * q + 1], w1, fmaf(xs[r][kk + 2 * q], w0, acc[c][r]));
                    }
                }
            } else {
                for (int kk = lane; kk < kc; kk += 32) {
                    const float w = load_any(p.w, p.w_dt, wrow + kk);
#pragma unroll
                    for (int r = 0; r < BR_ROWS; ++r) acc[c][r] = fmaf(xs[r][kk], w, acc[c][r]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < BR_COLS / 8; ++c) {
        const int o = o0 + c;
#pragma unroll
        for (int r = 0; r < BR_ROWS; ++r) {
            float v = warp_sum(acc[c][r]);
            if (lane == 0 && o < p.O && r < p.T) {
                if (p.bias != nullptr) v += load_any(p.bias, p.bias_dt, (size_t)b * p.O + o);
                store_any(p.out, p.out_dt, (size_t)r * p.out_stride + (size_t)b * p.out_bs + o, v);
            }
        }
    }
}
}  // namespace

RS_EXPORT int rs_block_linear(const void* in, int in_dt, long in_stride, long in_bs, const void* w, int w_dt,
                              const void* bias, int bias_dt, void* out, int out_dt, long out_stride, long out_bs, int T,
                              int B, int O, int I, void* stream) {
    if (T <= 0 || B <= 0 || O <= 0) return 0;
    BlockLinearParams p{in, in_dt, in_stride, in_bs, w, w_dt, bias, bias_dt, out, out_dt, out_stride, out_bs, T, O, I};
    if (T <= BR_ROWS) {
        block_linear_rows_kernel<<<dim3((O + BR_COLS - 1) / BR_COLS, B), 256, 0, (cudaStream_t)stream>>>(p);
        return rs_launch_result();
    }
    dim3 grid((O + BL_BN - 1) / BL_BN, (T + BL_BM - 1) / BL_BM, B);
    block_linear_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
    return rs_launch_result();
}

// --------------------------------------------------------------------------- gated linear recurrence
// One thread per (sequence, channel) walks the sequence's tokens of this step in order:
//   r = sigmoid(gates[t, g(c)]), i = sigmoid(gates[t, g(c) + bw]) with g(c) = (c / bw) * 2 bw + c % bw (the gates of a
//   block of bw channels lie together: its r, then its i), log a = -decay_c * r * softplus(lam[c]), a = exp(log a),
//   S = a S + sqrt(1 - a^2) i u[t, c];  out[t, c] = S * gelu_tanh(y[t, c] + y_bias[c]).
// S starts from the sequence's state slot (zero after admission) and is written back.
struct RecurrenceParams {
    const float* gates; long gates_stride;      // [T, 2W]: per block of bw channels, bw r pre-activations, then bw of i
    const float* u; long u_stride;              // [T, W]
    const float* y; long y_stride;              // [T, W] pre-activation of the gating branch
    const void* y_bias; int y_bias_dt;
    const void* lam; int lam_dt;
    void* out; int out_dt; long out_stride;
    float* state; long state_stride;
    const int* q_start; const int* slots;
    int W, n_seqs; float decay_c;
    int bw;                                     // channels per block of the gates' layout (W: all r, then all i)
};

__device__ __forceinline__ int gate_index(const RecurrenceParams& p, int c) { return (c / p.bw) * 2 * p.bw + c % p.bw; }

__global__ void gated_linear_recurrence_kernel(const RecurrenceParams p) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)p.n_seqs * p.W) return;
    const int s = (int)(idx / p.W), c = (int)(idx % p.W);
    const int row0 = p.q_start[s], n = p.q_start[s + 1] - row0;
    float* sp = p.state + (size_t)p.slots[s] * p.state_stride + c;
    float S = *sp;
    const float k = -p.decay_c * softplus_f32(load_any(p.lam, p.lam_dt, c));
    const float yb = p.y_bias != nullptr ? load_any(p.y_bias, p.y_bias_dt, c) : 0.f;
    const int gi = gate_index(p, c);
    for (int li = 0; li < n; ++li) {
        const size_t t = (size_t)(row0 + li);
        const float r = sigmoid_f32(p.gates[t * p.gates_stride + gi]);
        const float ig = sigmoid_f32(p.gates[t * p.gates_stride + gi + p.bw]);
        const float log_a = k * r;
        const float a = expf(log_a);
        const float m = sqrtf(-expm1f(2.0f * log_a));         // sqrt(1 - a^2) without cancellation near a = 1
        S = fmaf(a, S, m * ig * p.u[t * p.u_stride + c]);
        store_any(p.out, p.out_dt, t * p.out_stride + c, S * gelu_tanh_f32(p.y[t * p.y_stride + c] + yb));
    }
    *sp = S;
}

// The same recurrence for long portions, in three kernels.  The host cuts every sequence's tokens of the step into
// chunks of at most RS_SCAN_CHUNK (chunk_seq[k], chunk_start[k]: sequence and first local token; the chunks of a
// sequence are consecutive, seq_first_chunk[s] .. seq_first_chunk[s + 1]).  (1) a thread per (chunk, channel) runs the
// chunk from S = 0 and leaves the chunk's map S_out = A S_in + B (A the product of its a_t); (2) a thread per
// (sequence, channel) walks the sequence's chunks in order, leaves every chunk's S_in and the final S in the state;
// (3) a thread per (chunk, channel) runs the chunk again from its S_in and writes the outputs.
struct ScanChunks {
    const int* chunk_seq; const int* chunk_start; const int* seq_first_chunk;
    int n_chunks, chunk_len;
    float* work;                                  // [3][n_chunks][W]: A, B, S_in
};

__device__ __forceinline__ void recurrence_terms(const RecurrenceParams& p, size_t t, int c, float k, float& a, float& b) {
    const int gi = gate_index(p, c);
    const float r = sigmoid_f32(p.gates[t * p.gates_stride + gi]);
    const float ig = sigmoid_f32(p.gates[t * p.gates_stride + gi + p.bw]);
    const float log_a = k * r;
    a = expf(log_a);
    b = sqrtf(-expm1f(2.0f * log_a)) * ig * p.u[t * p.u_stride + c];
}

template <int PHASE>
__global__ void recurrence_chunk_kernel(const RecurrenceParams p, const ScanChunks sc) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)sc.n_chunks * p.W) return;
    const int ch = (int)(idx / p.W), c = (int)(idx % p.W);
    const int s = sc.chunk_seq[ch], l0 = sc.chunk_start[ch];
    const int row0 = p.q_start[s], n = min(sc.chunk_len, p.q_start[s + 1] - row0 - l0);
    const float k = -p.decay_c * softplus_f32(load_any(p.lam, p.lam_dt, c));
    const size_t slot = (size_t)ch * p.W + c, plane = (size_t)sc.n_chunks * p.W;
    if (PHASE == 1) {
        float A = 1.f, B = 0.f;
#pragma unroll 4
        for (int li = 0; li < n; ++li) {
            float a, b;
            recurrence_terms(p, (size_t)(row0 + l0 + li), c, k, a, b);
            A *= a;
            B = fmaf(a, B, b);
        }
        sc.work[slot] = A;
        sc.work[plane + slot] = B;
    } else {
        float S = sc.work[2 * plane + slot];
        const float yb = p.y_bias != nullptr ? load_any(p.y_bias, p.y_bias_dt, c) : 0.f;
#pragma unroll 4
        for (int li = 0; li < n; ++li) {
            const size_t t = (size_t)(row0 + l0 + li);
            float a, b;
            recurrence_terms(p, t, c, k, a, b);
            S = fmaf(a, S, b);
            store_any(p.out, p.out_dt, t * p.out_stride + c, S * gelu_tanh_f32(p.y[t * p.y_stride + c] + yb));
        }
    }
}

__global__ void recurrence_carry_kernel(const RecurrenceParams p, const ScanChunks sc) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)p.n_seqs * p.W) return;
    const int s = (int)(idx / p.W), c = (int)(idx % p.W);
    float* sp = p.state + (size_t)p.slots[s] * p.state_stride + c;
    float S = *sp;
    const size_t plane = (size_t)sc.n_chunks * p.W;
    for (int ch = sc.seq_first_chunk[s]; ch < sc.seq_first_chunk[s + 1]; ++ch) {
        const size_t slot = (size_t)ch * p.W + c;
        sc.work[2 * plane + slot] = S;
        S = fmaf(sc.work[slot], S, sc.work[plane + slot]);
    }
    *sp = S;
}

RS_EXPORT int rs_gated_linear_recurrence_chunked(const float* gates, long gates_stride, const float* u, long u_stride,
                                                 const float* y, long y_stride, const void* y_bias, int y_bias_dt,
                                                 const void* lam, int lam_dt, void* out, int out_dt, long out_stride,
                                                 float* state, long state_stride, const int* q_start, const int* slots,
                                                 int W, int n_seqs, float decay_c, int bw, const int* chunk_seq,
                                                 const int* chunk_start, const int* seq_first_chunk, int n_chunks,
                                                 int chunk_len, float* work, void* stream) {
    if (n_seqs <= 0 || W <= 0 || n_chunks <= 0) return 0;
    RecurrenceParams p{gates, gates_stride, u, u_stride, y, y_stride, y_bias, y_bias_dt, lam, lam_dt, out, out_dt,
                       out_stride, state, state_stride, q_start, slots, W, n_seqs, decay_c, bw > 0 ? bw : W};
    ScanChunks sc{chunk_seq, chunk_start, seq_first_chunk, n_chunks, chunk_len, work};
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned gc = (unsigned)(((long)n_chunks * W + 127) / 128), gs = (unsigned)(((long)n_seqs * W + 127) / 128);
    recurrence_chunk_kernel<1><<<gc, 128, 0, s>>>(p, sc);
    recurrence_carry_kernel<<<gs, 128, 0, s>>>(p, sc);
    recurrence_chunk_kernel<2><<<gc, 128, 0, s>>>(p, sc);
    return rs_launch_result();
}

RS_EXPORT int rs_gated_linear_recurrence(const float* gates, long gates_stride, const float* u, long u_stride, const float* y,
                                         long y_stride, const void* y_bias, int y_bias_dt, const void* lam, int lam_dt,
                                         void* out, int out_dt, long out_stride, float* state, long state_stride,
                                         const int* q_start, const int* slots, int W, int n_seqs, float decay_c, int bw,
                                         void* stream) {
    if (n_seqs <= 0 || W <= 0) return 0;
    RecurrenceParams p{gates, gates_stride, u, u_stride, y, y_stride, y_bias, y_bias_dt, lam, lam_dt, out, out_dt,
                       out_stride, state, state_stride, q_start, slots, W, n_seqs, decay_c, bw > 0 ? bw : W};
    const long total = (long)n_seqs * W;
    gated_linear_recurrence_kernel<<<(unsigned)((total + 127) / 128), 128, 0, (cudaStream_t)stream>>>(p);
    return rs_launch_result();
}

// --------------------------------------------------------------------------- latent key/value write + query rotation
// dkv: [T, rank + rot] float32 (the down-projection of the step's tokens).  Per token:
//   cache row = [ dkv[:rank] * rsqrt(mean^2 + eps) * norm_w | rotate(dkv[rank:]) | zeros up to lat ]
// written to cache[page][slot in page][lat] (one plane, one head), page from the block table at the token's position;
// and for every head h: q_lat[t, h * lat + rank + j] = rotate(q[t, h * q_head + q_nope + j]) for j < rot, zeros up to lat.
// The rotation turns the pairs (2i, 2i + 1), i < n_rot / 2, by the angle whose cosine and sine lie in
// cos_sin[position][i] and cos_sin[position][n_rot / 2 + i]; coordinates from n_rot on pass unchanged.
struct LatentParams {
    const float* dkv; long dkv_stride;
    const void* norm_w; int norm_dt; float eps;
    const void* q; int q_dt; long q_stride; int q_head, q_nope;
    void* q_lat; int q_lat_dt; long q_lat_stride;
    const float* cos_sin; int n_rot, table_rows;
    const int* positions; int pos_stride;
    const int* seq_of_token; const int* block_table; int table_stride, page_size;
    void* cache; int cache_dt; long page_stride; int num_pages;
    int rank, rot, lat, heads, n_tokens;
    int* status;
};

__device__ __forceinline__ float rotated(const LatentParams& p, const float* cs, float own, float partner, int j) {
    // j: index within the rotated part; own = v[j], partner = v[j ^ 1]
    if (cs == nullptr || j >= p.n_rot) return own;
    const int i = j >> 1, half = p.n_rot >> 1;
    const float c = cs[i], s = cs[half + i];
    return (j & 1) ? fmaf(own, c, partner * s) : fmaf(own, c, -partner * s);
}

__global__ void latent_kv_write_kernel(const LatentParams p) {
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int pos = p.positions[(size_t)t * p.pos_stride];
    const float* cs = nullptr;
    if (p.cos_sin != nullptr) {
        if (pos < 0 || pos >= p.table_rows) {
            if (threadIdx.x == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);
            return;
        }
        cs = p.cos_sin + (size_t)pos * p.n_rot;
    }
    // queries: the rotated part of every head
    for (int i = threadIdx.x; i < p.heads * (p.lat - p.rank); i += blockDim.x) {
        const int h = i / (p.lat - p.rank), j = i % (p.lat - p.rank);
        float v = 0.f;
        if (j < p.rot) {
            const size_t base = (size_t)t * p.q_stride + (size_t)h * p.q_head + p.q_nope;
            const float own = load_any(p.q, p.q_dt, base + j);
            const float partner = (j < p.n_rot) ? load_any(p.q, p.q_dt, base + (j ^ 1)) : 0.f;
            v = rotated(p, cs, own, partner, j);
        }
        store_any(p.q_lat, p.q_lat_dt, (size_t)t * p.q_lat_stride + (size_t)h * p.lat + p.rank + j, v);
    }
    if (p.cache == nullptr) return;
    const int page = p.block_table[(size_t)p.seq_of_token[t] * p.table_stride + pos / p.page_size];
    if (page < 0 || page >= p.num_pages) {
        if (threadIdx.x == 0) atomicOr(p.status, RS_STATUS_BAD_PAGE);
        return;
    }
    const float* row = p.dkv + (size_t)t * p.dkv_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.rank; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = block_sum(ss, scratch);
    const float s = 1.0f / sqrtf(ss / (float)p.rank + p.eps);
    const size_t dst = (size_t)page * p.page_stride + (size_t)(pos % p.page_size) * p.lat;
    for (int i = threadIdx.x; i < p.lat; i += blockDim.x) {
        float v = 0.f;
        if (i < p.rank) v = row[i] * s * load_any(p.norm_w, p.norm_dt, i);
        else if (i < p.rank + p.rot) {
            const int j = i - p.rank;
            v = rotated(p, cs, row[i], (j < p.n_rot) ? row[p.rank + (j ^ 1)] : 0.f, j);
        }
        store_any(p.cache, p.cache_dt, dst + i, v);
    }
}

RS_EXPORT int rs_latent_kv_write(const float* dkv, long dkv_stride, const void* norm_w, int norm_dt, float eps, const void* q,
                                 int q_dt, long q_stride, int q_head, int q_nope, void* q_lat, int q_lat_dt,
                                 long q_lat_stride, const float* cos_sin, int n_rot, int table_rows, const int* positions,
                                 int pos_stride, const int* seq_of_token, const int* block_table, int table_stride,
                                 int page_size, void* cache, int cache_dt, long page_stride, int num_pages, int rank, int rot,
                                 int lat, int heads, int n_tokens, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (n_rot % 2 || n_rot > rot || rank + rot > lat) return (int)cudaErrorInvalidValue;
    LatentParams p{dkv, dkv_stride, norm_w, norm_dt, eps, q, q_dt, q_stride, q_head, q_nope, q_lat, q_lat_dt, q_lat_stride,
                   cos_sin, n_rot, table_rows, positions, pos_stride, seq_of_token, block_table, table_stride, page_size,
                   cache, cache_dt, page_stride, num_pages, rank, rot, lat, heads, n_tokens, status};
    latent_kv_write_kernel<<<n_tokens, 128, 0, (cudaStream_t)stream>>>(p);
    return rs_launch_result();
}

// --------------------------------------------------------------------------- a gate per head
// a[t, h * dv + d] *= sigmoid(g[t, h]) in place; g float32 (pre-activations), the sigmoid in float32
__global__ void head_sigmoid_gate_kernel(void* __restrict__ a, int dt, long a_stride, const float* __restrict__ g, long g_stride,
                                         int heads, int dv, long n) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int w = heads * dv;
    const long t = idx / w;
    const int c = (int)(idx % w);
    const float z = g[t * g_stride + c / dv];
    const size_t at = (size_t)t * a_stride + c;
    store_any(a, dt, at, load_any(a, dt, at) * (1.0f / (1.0f + expf(-z))));
}

// the same with 16 bytes per thread: eight bfloat16 or four float32 values of one head (dv a multiple of that many,
// rows and the pointer aligned to 16 bytes)
template <typename T>
__global__ void head_sigmoid_gate_vec_kernel(T* __restrict__ a, long a_stride, const float* __restrict__ g, long g_stride,
                                             int heads, int dv, long n_pieces) {
    constexpr int V = 16 / sizeof(T);
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_pieces) return;
    const int per_row = heads * dv / V;
    const long t = idx / per_row;
    const int c = (int)(idx % per_row) * V;
    const float s = 1.0f / (1.0f + expf(-g[t * g_stride + c / dv]));
    uint4* at = reinterpret_cast<uint4*>(a + (size_t)t * a_stride + c);
    uint4 raw = *at;
    T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] = from_f32<T>(to_f32<T>(v[i]) * s);
    *at = raw;
}

RS_EXPORT int rs_head_sigmoid_gate(void* a, int dt, long a_stride, const float* g, long g_stride, int heads, int dv,
                                   int n_tokens, void* stream) {
    const long n = (long)n_tokens * heads * dv;
    if (n <= 0) return 0;
    const int v = dt == RS_F32 ? 4 : 8;
    if ((dt == RS_F32 || dt == RS_BF16) && dv % v == 0 && a_stride % v == 0 && (uintptr_t)a % 16 == 0) {
        const long pieces = n / v;
        RS_DISPATCH_DTYPE(dt, T, (head_sigmoid_gate_vec_kernel<T><<<(unsigned)((pieces + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            reinterpret_cast<T*>(a), a_stride, g, g_stride, heads, dv, pieces)));
        return rs_launch_result();
    }
    head_sigmoid_gate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, dt, a_stride, g, g_stride, heads,
                                                                                           dv, n);
    return rs_launch_result();
}

// --------------------------------------------------------------------------- activations
// out[r, c] = relu(in[r, c])^2
__global__ void relu_squared_kernel(const void* __restrict__ in, int dt, long in_stride, void* __restrict__ out,
                                    long out_stride, int rows, int n) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)rows * n) return;
    const int r = (int)(idx / n), c = (int)(idx % n);
    const float v = fmaxf(load_any(in, dt, (size_t)r * in_stride + c), 0.f);
    store_any(out, dt, (size_t)r * out_stride + c, v * v);
}

RS_EXPORT int rs_relu_squared(const void* in, int dt, long in_stride, void* out, long out_stride, int rows, int n,
                              void* stream) {
    if (rows <= 0 || n <= 0) return 0;
    const long total = (long)rows * n;
    relu_squared_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(in, dt, in_stride, out, out_stride,
                                                                                       rows, n);
    return rs_launch_result();
}
