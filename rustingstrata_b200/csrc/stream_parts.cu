// Parts of decoders that keep several residual streams and sum several embedding tables, for both engines:
//   * embed_sum: token row + a row chosen by a hash of (previous token, token) + a learned position row, written
//     to every residual stream; the previous token of a request's next portion lives in its state slot;
//   * stream_layernorm: layer norm (weight and bias) of a weighted sum of the residual streams of a token;
//   * stream_update: all streams at once from the old ones, x_t <- sum_s mix[s, t] x_s + out[t] y, and in the same
//     pass the layer norm of the next reader's weighted sum;
//   * router_topk: softmax or sigmoid over expert logits, choice by score + correction (within the best groups of
//     experts, if they form groups), weights from the uncorrected scores
//     of the chosen experts divided by their sum.
// Everything here is float32 whatever the activation type is; a token's row is computed in an order that only the
// row's own width fixes, never the batch.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int MAX_STREAMS = 16;

__device__ __forceinline__ void store_any(void* p, int dt, size_t i, float v) {
    if (dt == RS_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

struct EmbedSumParams {
    const void* tok; int tok_dt; int V;
    const void* bigram; int bigram_dt; int buckets; long mul_prev, mul_cur;      // bigram == null: no such table
    const void* pos; int pos_dt; int n_pos;                                       // pos == null: no position table
    const int* ids; const int* positions; int pos_stride; const int* seq_of_token; const int* q_start; const int* slots;
    const int* prev_state; long state_stride;
    float* out; long out_stride; int copies; int D;
    int* status;
    float tok_scale;                     // the token row is multiplied by it
};

__global__ void embed_sum_kernel(const EmbedSumParams p) {
    const int t = blockIdx.x;
    int id = p.ids[t];
    if (id < 0 || id >= p.V) {
        if (threadIdx.x == 0) atomicOr(p.status, RS_STATUS_BAD_TOKEN);
        id = 0;
    }
    const int s = p.seq_of_token[t];
    int place = p.positions[(size_t)t * p.pos_stride];
    long row = -1;
    if (p.bigram != nullptr) {
        if (place == 0) {
            row = p.buckets;                                   // a sequence's first token has a row of its own
        } else {
            int prev = t > p.q_start[s] ? p.ids[t - 1] : p.prev_state[(size_t)p.slots[s] * p.state_stride];
            if (prev < 0 || prev >= p.V) prev = 0;
            row = ((long)prev * p.mul_prev + (long)id * p.mul_cur) % (long)p.buckets;
            if (row < 0) row += p.buckets;                     // the remainder of a floored division, also for negative factors
        }
    }
    if (p.pos != nullptr && (place < 0 || place >= p.n_pos)) {
        if (threadIdx.x == 0) atomicOr(p.status, RS_STATUS_BAD_TOKEN);
        place = 0;
    }
    float* o = p.out + (size_t)t * p.out_stride;
    for (int i = threadIdx.x; i < p.D; i += blockDim.x) {
        float v = load_any(p.tok, p.tok_dt, (size_t)id * p.D + i) * p.tok_scale;
        if (row >= 0) v += load_any(p.bigram, p.bigram_dt, (size_t)row * p.D + i);
        if (p.pos != nullptr) v += load_any(p.pos, p.pos_dt, (size_t)place * p.D + i);
        for (int c = 0; c < p.copies; ++c) o[(size_t)c * p.D + i] = v;
    }
}

// the last token of every sequence of the step becomes its "previous token"; runs after embed_sum has read the old one
__global__ void store_last_token_kernel(const int* __restrict__ ids, const int* __restrict__ q_start,
                                        const int* __restrict__ slots, int* __restrict__ state, long state_stride,
                                        int n_seqs) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_seqs) return;
    state[(size_t)slots[s] * state_stride] = ids[q_start[s + 1] - 1];
}

struct StreamNormParams {
    const float* x; long x_stride; const int* rows;       // [tokens, S * D]; rows: which token each output row reads
    const void* coef; int coef_dt;                         // [S] or null: every stream counts once
    const void* w; int w_dt; const void* b; int b_dt; float eps;
    void* out; int out_dt; long out_stride;
    int S, D;
};

// mean and variance over u[0 .. D), held in shared memory; two passes, the variance from the deviations
__device__ __forceinline__ void layernorm_row(const float* u, int D, const void* w, int w_dt, const void* b, int b_dt,
                                              float eps, void* out, int out_dt, size_t out_base, float* scratch) {
    float sum = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) sum += u[i];
    const float mean = block_sum(sum, scratch) / (float)D;
    float sq = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { const float d = u[i] - mean; sq = fmaf(d, d, sq); }
    const float var = block_sum(sq, scratch) / (float)D;
    const float r = 1.0f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = (u[i] - mean) * r * load_any(w, w_dt, i);
        if (b != nullptr) v += load_any(b, b_dt, i);
        store_any(out, out_dt, out_base + i, v);
    }
}

__global__ void stream_layernorm_kernel(const StreamNormParams p) {
    extern __shared__ float u[];
    __shared__ float scratch[33];
    __shared__ float cf[MAX_STREAMS];
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < p.S; i += blockDim.x) cf[i] = p.coef != nullptr ? load_any(p.coef, p.coef_dt, i) : 1.0f;
    __syncthreads();
    const float* xr = p.x + (size_t)(p.rows != nullptr ? p.rows[r] : r) * p.x_stride;
    for (int i = threadIdx.x; i < p.D; i += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < p.S; ++s) v = fmaf(cf[s], xr[(size_t)s * p.D + i], v);
        u[i] = v;
    }
    __syncthreads();
    layernorm_row(u, p.D, p.w, p.w_dt, p.b, p.b_dt, p.eps, p.out, p.out_dt, (size_t)r * p.out_stride, scratch);
}

struct StreamUpdateParams {
    float* x; long x_stride;                               // [tokens, S * D], updated in place
    const float* y; long y_stride;                         // the sublayer's output [tokens, D]
    const void* mix; int mix_dt;                           // [S, S], indexed [from, to]
    const void* outc; int outc_dt;                         // [S]
    StreamNormParams next;                                 // next.out != null: the next reader's norm in the same pass
    int S, D;
};

// MS: the least of 1, 2, 4, 8, 16 that holds the S streams (the loops over streams are unrolled to it)
template <int MS>
__global__ void stream_update_kernel(const StreamUpdateParams p) {
    extern __shared__ float u[];
    __shared__ float scratch[33];
    __shared__ float mx[MAX_STREAMS * MAX_STREAMS], oc[MAX_STREAMS], cf[MAX_STREAMS];
    const int r = blockIdx.x, S = p.S;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) mx[i] = load_any(p.mix, p.mix_dt, i);
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        oc[i] = load_any(p.outc, p.outc_dt, i);
        cf[i] = p.next.coef != nullptr ? load_any(p.next.coef, p.next.coef_dt, i) : 1.0f;
    }
    __syncthreads();
    float* xr = p.x + (size_t)r * p.x_stride;
    const float* yr = p.y + (size_t)r * p.y_stride;
    const bool norm = p.next.out != nullptr;
    for (int i = threadIdx.x; i < p.D; i += blockDim.x) {
        float xs[MS];
#pragma unroll
        for (int s = 0; s < MS; ++s) xs[s] = s < S ? xr[(size_t)s * p.D + i] : 0.f;
        const float yv = yr[i];
        float acc = 0.f;
#pragma unroll
        for (int t = 0; t < MS; ++t) {
            if (t >= S) break;
            float nx = 0.f;
#pragma unroll
            for (int s = 0; s < MS; ++s)
                if (s < S) nx = fmaf(mx[s * S + t], xs[s], nx);
            nx = fmaf(oc[t], yv, nx);
            xr[(size_t)t * p.D + i] = nx;
            acc = fmaf(cf[t], nx, acc);
        }
        if (norm) u[i] = acc;
    }
    if (!norm) return;
    __syncthreads();
    layernorm_row(u, p.D, p.next.w, p.next.w_dt, p.next.b, p.next.b_dt, p.next.eps, p.next.out, p.next.out_dt,
                  (size_t)r * p.next.out_stride, scratch);
}

// one warp per token: scores = softmax(logits), or sigmoid(logits) each for itself (``sigmoid``); the `top` largest of
// scores + correction are chosen (the lower index on a tie); with ``n_groups`` > 0 the experts form that many equal
// groups of neighbours, a group is worth the sum of its two largest scores + correction, and only experts of the
// ``keep`` groups worth most can be chosen (the lower index on a tie); weights = the chosen experts' scores times
// ``scale``, divided by (their sum + 1e-20) first when ``renorm`` is set
__global__ void router_topk_kernel(const float* __restrict__ logits, long l_stride, const void* __restrict__ corr,
                                   int corr_dt, int E, int top, int n_tokens, int sigmoid, int n_groups, int keep, float scale,
                                   int renorm, int* __restrict__ choice, float* __restrict__ weight, int* status) {
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int t = blockIdx.x * wpb + warp;
    if (t >= n_tokens) return;
    float* score = sm + (size_t)warp * (2 * E + 2 * n_groups);
    float* pick = score + E;
    float* worth = pick + E;                 // [n_groups]
    float* kept = worth + n_groups;          // [n_groups] 1: the group's experts can be chosen
    const float* z = logits + (size_t)t * l_stride;
    if (sigmoid) {
        bool bad = false;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            bad |= !isfinite(v);
            score[e] = 1.0f / (1.0f + expf(-v));
        }
        if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(status, RS_STATUS_NON_FINITE);
    } else {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float v = expf(z[e] - m); score[e] = v; sum += v; }
        sum = warp_sum(sum);
        if (!(sum > 0.f) || !isfinite(sum)) { if (lane == 0) atomicOr(status, RS_STATUS_NON_FINITE); }
        for (int e = lane; e < E; e += 32) score[e] = score[e] / sum;
    }
    for (int e = lane; e < E; e += 32) pick[e] = corr != nullptr ? score[e] + load_any(corr, corr_dt, e) : score[e];
    __syncwarp();
    if (n_groups > 0) {
        const int per = E / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;              // the group's largest and second largest
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = pick[e];
                if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
            }
            worth[g] = per > 1 ? a + b : a;
            kept[g] = 0.f;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY; int bi = 0x7FFFFFFF;
            for (int g = lane; g < n_groups; g += 32) { const float v = worth[g]; if (kept[g] == 0.f && (v > best || bi == 0x7FFFFFFF)) { best = v; bi = g; } }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7FFFFFFF && (bi == 0x7FFFFFFF || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
            }
            if (bi >= 0 && bi < n_groups && lane == 0) kept[bi] = 1.f;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (kept[e / per] == 0.f) pick[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY; int bi = 0x7FFFFFFF;
        for (int e = lane; e < E; e += 32) { const float v = pick[e]; if (v > best) { best = v; bi = e; } }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi < 0 || bi >= E) bi = 0;                           // nothing finite left: every lane agrees
        const float s = score[bi];
        total += s;
        if (lane == 0) { choice[(size_t)t * top + k] = bi; weight[(size_t)t * top + k] = s; pick[bi] = -INFINITY; }
        __syncwarp();
    }
    const float f = renorm ? scale / (total + 1e-20f) : scale;
    __syncwarp();
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= f;
}
}  // namespace

RS_EXPORT int rs_embed_sum(const void* tok, int tok_dt, int V, const void* bigram, int bigram_dt, int buckets, long mul_prev,
                           long mul_cur, const void* pos, int pos_dt, int n_pos, const int* ids, const int* positions,
                           int pos_stride, const int* seq_of_token, const int* q_start, const int* slots, int* prev_state,
                           long state_stride, float* out, long out_stride, int copies, int D, int n_tokens, int n_seqs,
                           float tok_scale, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (bigram != nullptr && (buckets <= 0 || prev_state == nullptr)) return (int)cudaErrorInvalidValue;
    EmbedSumParams p{tok, tok_dt, V, bigram, bigram_dt, buckets, mul_prev, mul_cur, pos, pos_dt, n_pos, ids, positions,
                     pos_stride, seq_of_token, q_start, slots, prev_state, state_stride, out, out_stride, copies, D, status, tok_scale};
    cudaStream_t s = (cudaStream_t)stream;
    embed_sum_kernel<<<n_tokens, D >= 1024 ? 256 : 128, 0, s>>>(p);
    int e = rs_launch_result();
    if (e != 0 || bigram == nullptr) return e;
    store_last_token_kernel<<<(n_seqs + 127) / 128, 128, 0, s>>>(ids, q_start, slots, prev_state, state_stride, n_seqs);
    return rs_launch_result();
}

namespace {
int norm_threads(int D) { return D >= 4096 ? 512 : (D >= 1024 ? 256 : 128); }
}

RS_EXPORT int rs_stream_layernorm(const float* x, long x_stride, const int* rows, const void* coef, int coef_dt,
                                  const void* w, int w_dt, const void* b, int b_dt, float eps, void* out, int out_dt,
                                  long out_stride, int S, int D, int n_rows, void* stream) {
    if (n_rows <= 0) return 0;
    if (S <= 0 || S > MAX_STREAMS || D <= 0 || (size_t)D * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    StreamNormParams p{x, x_stride, rows, coef, coef_dt, w, w_dt, b, b_dt, eps, out, out_dt, out_stride, S, D};
    stream_layernorm_kernel<<<n_rows, norm_threads(D), (size_t)D * sizeof(float), (cudaStream_t)stream>>>(p);
    return rs_launch_result();
}

RS_EXPORT int rs_stream_update(float* x, long x_stride, const float* y, long y_stride, const void* mix, int mix_dt,
                               const void* outc, int outc_dt, const void* coef, int coef_dt, const void* w, int w_dt,
                               const void* b, int b_dt, float eps, void* out, int out_dt, long out_stride, int S, int D,
                               int n_rows, void* stream) {
    if (n_rows <= 0) return 0;
    if (S <= 0 || S > MAX_STREAMS || D <= 0 || (size_t)D * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    StreamUpdateParams p;
    p.x = x; p.x_stride = x_stride; p.y = y; p.y_stride = y_stride; p.mix = mix; p.mix_dt = mix_dt; p.outc = outc;
    p.outc_dt = outc_dt; p.S = S; p.D = D;
    p.next = StreamNormParams{x, x_stride, nullptr, coef, coef_dt, w, w_dt, b, b_dt, eps, out, out_dt, out_stride, S, D};
    const int threads = S > 8 && norm_threads(D) > 256 ? 256 : norm_threads(D);     // the widest form holds 16 streams in registers
    const size_t smem = out != nullptr ? (size_t)D * sizeof(float) : 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (S == 1) stream_update_kernel<1><<<n_rows, threads, smem, st>>>(p);
    else if (S == 2) stream_update_kernel<2><<<n_rows, threads, smem, st>>>(p);
    else if (S <= 4) stream_update_kernel<4><<<n_rows, threads, smem, st>>>(p);
    else if (S <= 8) stream_update_kernel<8><<<n_rows, threads, smem, st>>>(p);
    else stream_update_kernel<16><<<n_rows, threads, smem, st>>>(p);
    return rs_launch_result();
}

RS_EXPORT int rs_router_topk(const float* logits, long l_stride, const void* corr, int corr_dt, int E, int top, int n_tokens,
                             int sigmoid, int n_groups, int keep, float scale, int renorm, int* choice, float* weight, int* status,
                             void* stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || E > 1024) return (int)cudaErrorInvalidValue;
    if (n_groups < 0 || (n_groups > 0 && (E % n_groups || keep < 1 || keep > n_groups || top > keep * (E / n_groups))))
        return (int)cudaErrorInvalidValue;
    const int wpb = 4;
    router_topk_kernel<<<(n_tokens + wpb - 1) / wpb, wpb * 32, (size_t)wpb * (2 * E + 2 * n_groups) * sizeof(float),
                         (cudaStream_t)stream>>>(
        logits, l_stride, corr, corr_dt, E, top, n_tokens, sigmoid, n_groups, keep, scale, renorm, choice, weight, status);
    return rs_launch_result();
}
