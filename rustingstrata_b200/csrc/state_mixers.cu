// Mixers that keep a matrix of state per head instead of a cache of keys, for both engines:
//   * state_recurrence: per (sequence, head) a [rows, columns] float32 state walked token by token, in two forms:
//       gated write   S = diag(g) S + w v^T,                                    o = S^T q      (HGRN2: g = f, w = 1 - f)
//       delta rule    S = diag(g) S;  u = beta (v - S^T k);  S = S + k u^T;     o = S^T q      (decay per key channel)
//   * hgrn2_prep: q = silu(.), forget gate with a lower bound, both laid out in padded rows;
//   * retention_prep: q and k rotated by position (halves of the rotated prefix paired), k scaled, in padded rows;
//   * delta_prep: short convolution over time + silu on q, k, v; unit-length q and k; decay and write strength;
//   * conv_tail_update: a request's last taps - 1 projected rows after the step;
//   * head_norm_gate: every head's read-out divided by its root mean square, times a weight and a sigmoid or SiLU gate;
//   * activation: elementwise xIELU / tanh-GELU;  scale_rows: float32 rows times one number.
// Gates, decays, norms and the state are float32 whatever the engine's element type.
#include "common.cuh"
#include <math.h>

namespace {

__device__ __forceinline__ void store_any(void* p, int dt, size_t i, float v) {
    if (dt == RS_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------------------------------------ the recurrence
// A column of a head's state belongs to RL = 8 (16 in small steps) neighbouring lanes; each lane keeps RPT rows of it in
// registers, so a head has RL * RPT rows.  A warp walks 32 / RL columns, a CTA 8, 16 or 32.  Sums over rows are
// shuffles inside the RL lanes: no shared memory and no barrier in the token loop, and an order of additions that
// depends on nothing but the head's shape and RL.  In a request's slot a head's state is stored column by column ([column][padded rows]), so the
// loads and stores at both ends of a step are whole 16-byte runs.
constexpr int ROW_LANES = 8;
constexpr int COLS_PER_CTA = 32;

struct RecurrenceParams {
    const float* q; long q_stride;          // [T, q heads * rows_pad]
    const float* k; long k_stride;          // delta rule: keys [T, q heads * rows_pad]; gated write: w [T, heads * rows_pad]
    const float* g; long g_stride;          // [T, heads * rows_pad] decay of every row
    const float* beta; long beta_stride;    // [T, heads] (delta rule)
    const float* v; long v_stride;          // [T, heads * columns]
    float* out; long out_stride;            // [T, heads * columns]
    float* state; long state_stride;        // [slots, heads * columns * rows_pad]
    const int* q_start; const int* slots;
    int heads, group, columns;              // group: state heads per q/k head (delta rule)
};

template <int RL>
__device__ __forceinline__ float sum_row_lanes(float v) {
#pragma unroll
    for (int o = 1; o < RL; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Lane rl of a column keeps rows 4 RL i + 4 rl .. + 3 for i < RPT / 4: the lanes of a column read neighbouring bytes,
// from shared memory without bank conflicts and from the state in whole lines.
template <int RPT, int RL>
__device__ __forceinline__ void load_rows(const float* p, float* r) {
#pragma unroll
    for (int m = 0; m < RPT; m += 4) {
        const float4 a = *reinterpret_cast<const float4*>(p + m * RL);
        r[m] = a.x; r[m + 1] = a.y; r[m + 2] = a.z; r[m + 3] = a.w;
    }
}

// The step's per-token inputs (q, k, g rows of the head, the CTA's 32 values, the write strength) reach the token loop
// through shared memory, a chunk of tokens at a time with cp.async, one chunk ahead of the one being walked: the loop
// itself waits for nothing but its own arithmetic.  For the delta rule both sums over rows of a token are taken from
// the decayed state S' = diag(g) S in one round of shuffles: with r = S'^T k and a = S'^T q, u = beta (v - r) and the
// read-out of S' + k u^T is a + u (k . q).
template <int RP_> struct RecurrenceStage {
    static constexpr int RP = RP_;
    static constexpr int CHUNK = RP_ <= 128 ? 16 : 8;                 // tokens per buffer
    static constexpr int ROW = 3 * RP + COLS_PER_CTA + 4;              // q | k | g | v of the CTA's columns | beta, pad
    static constexpr size_t BYTES = 2ull * CHUNK * ROW * sizeof(float);
};

__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int RPT, bool DELTA, int RL>
__global__ void __launch_bounds__(256) state_recurrence_kernel(RecurrenceParams p) {
    using St = RecurrenceStage<RPT * RL>;
    constexpr int RP = St::RP, CHUNK = St::CHUNK, ROW = St::ROW;
    extern __shared__ __align__(16) float stage[];         // [2][CHUNK][ROW]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rl = lane & (RL - 1), cl = lane / RL;
    const int s = blockIdx.x / p.heads, h = blockIdx.x % p.heads;
    const int nthreads = blockDim.x, cols_cta = blockDim.x / RL;             // a CTA walks 2 to 32 columns
    const int jl = warp * (32 / RL) + cl;                   // column within the CTA
    const int j = blockIdx.y * cols_cta + jl;
    const bool live = j < p.columns;
    const int jc = live ? j : p.columns - 1;              // lanes beyond the last column walk it too and store nothing
    const int t0 = p.q_start[s], t1 = p.q_start[s + 1];
    const int n = t1 - t0;
    float* sp = p.state + (size_t)p.slots[s] * p.state_stride + ((size_t)h * p.columns + jc) * RP + rl * 4;
    float S[RPT];
    load_rows<RPT, RL>(sp, S);
    const size_t q_off = (size_t)(DELTA ? h / p.group : h) * RP;
    const size_t k_off = DELTA ? q_off : (size_t)h * RP;
    const size_t g_off = (size_t)h * RP;

    // what this thread copies of every token: pieces tid, tid + threads, .. of the 3 RP / 4 16-byte pieces of q | k | g,
    // and one of the CTA's values or the write strength
    constexpr int PIECES = 3 * RP / 4, MAX_OWN = (PIECES + 63) / 64;
    const float* own_src[MAX_OWN];
    long own_step[MAX_OWN];
    int own_dst[MAX_OWN];
#pragma unroll
    for (int e = 0; e < MAX_OWN; ++e) {
        const int piece = tid + e * nthreads;
        const int which = piece / (RP / 4), off = (piece % (RP / 4)) * 4;
        own_dst[e] = piece < PIECES ? which * RP + off : -1;
        own_step[e] = which == 0 ? p.q_stride : which == 1 ? p.k_stride : p.g_stride;
        own_src[e] = (which == 0 ? p.q + q_off : which == 1 ? p.k + k_off : p.g + g_off) + (size_t)t0 * own_step[e] + off;
    }
    const bool own_v = tid < cols_cta, own_b = DELTA && tid == cols_cta;
    const float* small_src = own_v ? p.v + (size_t)t0 * p.v_stride + (size_t)h * p.columns + min((int)blockIdx.y * cols_cta + tid, p.columns - 1)
                                   : p.beta + (size_t)t0 * p.beta_stride + h;
    const long small_step = own_v ? p.v_stride : p.beta_stride;
    const int small_dst = 3 * RP + (own_v ? tid : COLS_PER_CTA);

    auto fetch = [&](int c) {                               // chunk c of the step's tokens into buffer c & 1
        float* dst = stage + (size_t)(c & 1) * CHUNK * ROW;
        const int first = c * CHUNK, count = min(CHUNK, n - c * CHUNK);
#pragma unroll
        for (int e = 0; e < MAX_OWN; ++e) {
            if (own_dst[e] < 0) continue;
            const float* src = own_src[e] + (size_t)first * own_step[e];
            for (int tt = 0; tt < count; ++tt) cp_async_16(dst + tt * ROW + own_dst[e], src + (size_t)tt * own_step[e]);
        }
        if (own_v || own_b) {
            const float* src = small_src + (size_t)first * small_step;
            for (int tt = 0; tt < count; ++tt) cp_async_4(dst + tt * ROW + small_dst, src + (size_t)tt * small_step);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const int chunks = (n + CHUNK - 1) / CHUNK;
    if (chunks > 0) fetch(0);
    for (int c = 0; c < chunks; ++c) {
        if (c + 1 < chunks) {
            fetch(c + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        float* buf = stage + (size_t)(c & 1) * CHUNK * ROW;
        const int count = min(CHUNK, n - c * CHUNK);
        if (DELTA) {                                        // k . q of every token of the chunk, once for all columns
            constexpr int TEAM = 4;                         // lanes per token, whatever the CTA's width: one order of additions
            const int tt = tid / TEAM, part = tid % TEAM;
            float d = 0.f;
            if (tt < count)
                for (int i = part; i < RP; i += TEAM) d = fmaf(buf[tt * ROW + i], buf[tt * ROW + RP + i], d);
#pragma unroll
            for (int o = TEAM / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            if (part == 0 && tt < count) buf[tt * ROW + 3 * RP + COLS_PER_CTA + 1] = d;
            __syncthreads();
        }
#pragma unroll 2
        for (int tt = 0; tt < count; ++tt) {
            const float* row = buf + tt * ROW;
            float qc[RPT], kc[RPT], gc[RPT];
            load_rows<RPT, RL>(row + rl * 4, qc);
            load_rows<RPT, RL>(row + RP + rl * 4, kc);
            load_rows<RPT, RL>(row + 2 * RP + rl * 4, gc);
            const float vc = row[3 * RP + jl];
            float acc;
            if (DELTA) {
                const float bc = row[3 * RP + COLS_PER_CTA], d = row[3 * RP + COLS_PER_CTA + 1];
                float r4[4] = {0.f, 0.f, 0.f, 0.f}, a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int m = 0; m < RPT; ++m) {
                    S[m] *= gc[m];
                    r4[m & 3] = fmaf(S[m], kc[m], r4[m & 3]);
                    a4[m & 3] = fmaf(S[m], qc[m], a4[m & 3]);
                }
                float r = (r4[0] + r4[1]) + (r4[2] + r4[3]);
                float a = (a4[0] + a4[1]) + (a4[2] + a4[3]);
                r = sum_row_lanes<RL>(r);
                a = sum_row_lanes<RL>(a);
                const float u = bc * (vc - r);
#pragma unroll
                for (int m = 0; m < RPT; ++m) S[m] = fmaf(kc[m], u, S[m]);
                acc = fmaf(u, d, a);
            } else {
                float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int m = 0; m < RPT; ++m) { S[m] = fmaf(gc[m], S[m], kc[m] * vc); a4[m & 3] = fmaf(S[m], qc[m], a4[m & 3]); }
                acc = sum_row_lanes<RL>((a4[0] + a4[1]) + (a4[2] + a4[3]));
            }
            if (rl == 0 && live) p.out[(size_t)(t0 + c * CHUNK + tt) * p.out_stride + (size_t)h * p.columns + j] = acc;
        }
        __syncthreads();                                    // the buffer is refilled two chunks on
    }
    if (live) {
#pragma unroll
        for (int m = 0; m < RPT; m += 4)
            *reinterpret_cast<float4*>(sp + m * RL) = make_float4(S[m], S[m + 1], S[m + 2], S[m + 3]);
    }
}

// ------------------------------------------------------------------------------------------------ HGRN2: gates
// proj [T, q (heads * dim) | f (heads * dim) | ...] float32: q = silu(.), f = l + (1 - l) sigmoid(. + bias);
// rows padded to rows_pad with zeros (a padded row of the state stays zero whatever it is multiplied by).
__global__ void hgrn2_prep_kernel(const float* proj, long proj_stride, const void* f_bias, int fb_dt, const void* lower, int lo_dt,
                                  float* q, float* g, float* w, int heads, int dim, int rows_pad, long n) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int i = (int)(idx % rows_pad);
    const int h = (int)((idx / rows_pad) % heads);
    const long t = idx / ((long)rows_pad * heads);
    float qv = 0.f, gv = 0.f, wv = 0.f;
    if (i < dim) {
        const int c = h * dim + i;
        const float* row = proj + t * proj_stride;
        qv = silu_f(row[c]);
        const float lo = load_any(lower, lo_dt, c);
        const float pre = row[heads * dim + c] + (f_bias ? load_any(f_bias, fb_dt, c) : 0.f);
        gv = lo + (1.0f - lo) * sigmoid_f(pre);
        wv = 1.0f - gv;
    }
    q[idx] = qv; g[idx] = gv; w[idx] = wv;
}

// proj [T, q (heads * dim) | k (heads * dim) | ...] float32: the first n_rot coordinates of every q and k head turned by
// the token's position, coordinate i < n_rot / 2 together with i + n_rot / 2 (cos_sin [positions, cos | sin]), k times
// k_scale afterwards; rows padded to rows_pad with zeros.
__global__ void retention_prep_kernel(const float* proj, long proj_stride, const float* cos_sin, int n_rot, int table_rows,
                                      const int* positions, int pos_stride, float k_scale, float* q, float* k, int heads, int dim,
                                      int rows_pad, long n, int* status) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int i = (int)(idx % rows_pad);
    const int h = (int)((idx / rows_pad) % heads);
    const long t = idx / ((long)rows_pad * heads);
    float qv = 0.f, kv = 0.f;
    if (i < dim) {
        const float* qrow = proj + t * proj_stride + (size_t)h * dim;
        const float* krow = qrow + (size_t)heads * dim;
        qv = qrow[i]; kv = krow[i];
        if (i < n_rot) {
            const int half = n_rot >> 1;
            const int pos = positions[t * pos_stride];
            if (pos >= table_rows && i == 0) atomicOr(status, RS_STATUS_BAD_PLAN);                // a position the table does not hold
            const float* cs = cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * n_rot;
            const int a = i < half ? i : i - half;
            const float c = cs[a], sn = cs[half + a];
            const int j = i < half ? i + half : i - half;
            const float sg = i < half ? -sn : sn;
            qv = fmaf(qv, c, qrow[j] * sg);
            kv = fmaf(kv, c, krow[j] * sg);
        }
        kv *= k_scale;
    }
    q[idx] = qv; k[idx] = kv;
}

// ------------------------------------------------------------------------------------------------ delta rule: inputs
constexpr int MAX_PER_LANE = 8;          // heads of up to 256 channels

struct DeltaPrepParams {
    const float* proj; long proj_stride;      // [T, q (qk heads * dim) | k (qk heads * dim) | v (heads * vdim) | beta (heads) | ...]
    const void* conv; int conv_dt;            // [taps, C] tap-major, C = the q, k and v channels; null with taps <= 1... or 0
    const float* tail; long tail_stride;      // [slots, (taps - 1) * C]
    const float* step; long step_stride;      // [T, heads * dim]: what the decay's softplus reads, before its bias
    const void* dt_bias; int dtb_dt;          // [heads * dim]
    const void* a_log; int al_dt;             // [heads]
    float* q; float* k; float* g;             // [T, qk heads * rows_pad] x 2, [T, heads * rows_pad]
    float* v; float* beta;                    // [T, heads * vdim], [T, heads]
    const int* seq_of_token; const int* q_start; const int* slots;
    int C, taps, qk_heads, heads, dim, vdim, rows_pad, beta_off, n_tokens;
    float unit_eps, q_scale;
};

// A warp per (token, item); items: the q heads, the k heads, the v heads, then one per head for decay and strength.
__global__ void __launch_bounds__(256) delta_prep_kernel(DeltaPrepParams p) {
    const int lane = threadIdx.x & 31;
    const int items = 2 * p.qk_heads + 2 * p.heads;
    const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (long)p.n_tokens * items) return;
    const int t = (int)(wid / items), item = (int)(wid % items);
    if (item >= 2 * p.qk_heads + p.heads) {               // decay of every key channel, and the write strength
        const int h = item - 2 * p.qk_heads - p.heads;
        const float rate = expf(load_any(p.a_log, p.al_dt, h));
        for (int i = lane; i < p.rows_pad; i += 32) {
            float gv = 0.f;
            if (i < p.dim) {
                const int c = h * p.dim + i;
                gv = expf(-rate * softplus_f(p.step[(size_t)t * p.step_stride + c] + load_any(p.dt_bias, p.dtb_dt, c)));
            }
            p.g[((size_t)t * p.heads + h) * p.rows_pad + i] = gv;
        }
        if (lane == 0) p.beta[(size_t)t * p.heads + h] = sigmoid_f(p.proj[(size_t)t * p.proj_stride + p.beta_off + h]);
        return;
    }
    int kind, base, width, head;
    if (item < p.qk_heads) { kind = 0; head = item; base = head * p.dim; width = p.dim; }
    else if (item < 2 * p.qk_heads) { kind = 1; head = item - p.qk_heads; base = (p.qk_heads + head) * p.dim; width = p.dim; }
    else { kind = 2; head = item - 2 * p.qk_heads; base = 2 * p.qk_heads * p.dim + head * p.vdim; width = p.vdim; }
    const int s = p.seq_of_token[t];
    const int t0 = p.q_start[s];
    const float* tail = p.tail ? p.tail + (size_t)p.slots[s] * p.tail_stride : nullptr;
    float acc[MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < MAX_PER_LANE; ++m) {
        const int d = lane + 32 * m;
        acc[m] = 0.f;
        if (d < width) {
            const int c = base + d;
            float a;
            if (p.taps >= 1 && p.conv) {
                a = 0.f;
                for (int jt = 0; jt < p.taps; ++jt) {
                    const int back = p.taps - 1 - jt;                  // how many tokens before t this tap reads
                    float x;
                    if (t - back >= t0) x = p.proj[(size_t)(t - back) * p.proj_stride + c];
                    else x = tail[(size_t)(p.taps - 1 - (t0 - (t - back))) * p.C + c];
                    a = fmaf(load_any(p.conv, p.conv_dt, (size_t)jt * p.C + c), x, a);
                }
            } else {
                a = p.proj[(size_t)t * p.proj_stride + c];
            }
            a = silu_f(a);
            acc[m] = a;
            ss = fmaf(a, a, ss);
        }
    }
    if (kind == 2) {
#pragma unroll
        for (int m = 0; m < MAX_PER_LANE; ++m) {
            const int d = lane + 32 * m;
            if (d < width) p.v[((size_t)t * p.heads + head) * p.vdim + d] = acc[m];
        }
        return;
    }
    ss = warp_sum(ss);
    const float r = (kind == 0 ? p.q_scale : 1.0f) / sqrtf(ss + p.unit_eps);
    float* dst = (kind == 0 ? p.q : p.k) + ((size_t)t * p.qk_heads + head) * p.rows_pad;
#pragma unroll
    for (int m = 0; m < MAX_PER_LANE; ++m) {
        const int d = lane + 32 * m;
        if (d < p.rows_pad) dst[d] = d < width ? acc[m] * r : 0.f;
    }
}

// After the step: a request's tail holds the last taps - 1 projected rows it has seen.  One thread per (sequence, channel)
// walks the tail from its oldest row on: what it reads lies at or after what it writes.
__global__ void conv_tail_update_kernel(const float* proj, long proj_stride, float* tail, long tail_stride, const int* q_start,
                                        const int* slots, int C, int taps, int n_seqs) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int s = (int)(idx / C), c = (int)(idx % C);
    const int t0 = q_start[s], t1 = q_start[s + 1], n = t1 - t0, keep = taps - 1;
    float* row = tail + (size_t)slots[s] * tail_stride;
    for (int e = 0; e < keep; ++e) {
        const int t = t1 - keep + e;
        row[(size_t)e * C + c] = t >= t0 ? proj[(size_t)t * proj_stride + c] : row[(size_t)(e + n) * C + c];
    }
}

// ------------------------------------------------------------------------------------------------ read-out
// A warp per (token, head): o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate) (weight and gate optional).
__global__ void __launch_bounds__(256) head_norm_gate_kernel(const float* o, long o_stride, const void* weight, int w_dt, const float* gate,
                                                            long gate_stride, void* out, int out_dt, long out_stride, int heads, int vdim,
                                                            float eps, int n_tokens, int gate_silu) {
    const int lane = threadIdx.x & 31;
    const long wid = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (long)n_tokens * heads) return;
    const int t = (int)(wid / heads), h = (int)(wid % heads);
    const float* row = o + (size_t)t * o_stride + (size_t)h * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) ss = fmaf(row[d], row[d], ss);
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int d = lane; d < vdim; d += 32) {
        float y = row[d] * r;
        if (weight) y *= load_any(weight, w_dt, d);
        if (gate) {
            const float z = gate[(size_t)t * gate_stride + (size_t)h * vdim + d];
            y *= gate_silu ? silu_f(z) : sigmoid_f(z);
        }
        store_any(out, out_dt, (size_t)t * out_stride + (size_t)h * vdim + d, y);
    }
}

// ------------------------------------------------------------------------------------------------ activations
enum Activation : int { ACT_XIELU = 0, ACT_GELU_TANH = 1 };

// xIELU with two learned numbers (p, q): z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
__device__ __forceinline__ float activate(float z, int kind, float ap, float an) {
    if (kind == ACT_XIELU) return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void activation_kernel(const T* x, long x_stride, T* out, long out_stride, int width, long n, int kind, const void* pq, int pq_dt) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const long t = idx / width; const int c = (int)(idx % width);
    float ap = 0.f, an = 0.f;
    if (kind == ACT_XIELU) { ap = softplus_f(load_any(pq, pq_dt, 0)); an = 0.5f + softplus_f(load_any(pq, pq_dt, 1)); }
    out[t * out_stride + c] = from_f32<T>(activate(to_f32<T>(x[t * x_stride + c]), kind, ap, an));
}

// 16 bytes per thread and step (rows that start on 16 bytes, a width that is a multiple of the 16 bytes' elements)
template <typename T>
__global__ void __launch_bounds__(256) activation_vec_kernel(const T* x, long x_stride, T* out, long out_stride, int width, int n_rows,
                                                             int kind, const void* pq, int pq_dt) {
    constexpr int V = 16 / sizeof(T);
    float ap = 0.f, an = 0.f;
    if (kind == ACT_XIELU) { ap = softplus_f(load_any(pq, pq_dt, 0)); an = 0.5f + softplus_f(load_any(pq, pq_dt, 1)); }
    const int per_row = width / V;
    const long total = (long)n_rows * per_row;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long t = i / per_row; const int c = (int)(i % per_row) * V;
        uint4 raw = *reinterpret_cast<const uint4*>(x + t * x_stride + c);
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int j = 0; j < V; ++j) e[j] = from_f32<T>(activate(to_f32<T>(e[j]), kind, ap, an));
        *reinterpret_cast<uint4*>(out + t * out_stride + c) = raw;
    }
}

__global__ void scale_rows_kernel(float* x, long stride, int width, long n, float scale) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    x[(idx / width) * stride + idx % width] *= scale;
}

}  // namespace

// ==================================================================================================== entry points
RS_EXPORT int rs_state_recurrence_rows_pad(int rows) {
    for (int rpt = 4; rpt <= 32; rpt *= 2) if (rows <= rpt * ROW_LANES) return rpt * ROW_LANES;
    return 0;
}

RS_EXPORT int rs_state_recurrence(const float* q, long q_stride, const float* k, long k_stride, const float* g, long g_stride,
                                  const float* beta, long beta_stride, const float* v, long v_stride, float* out, long out_stride,
                                  float* state, long state_stride, const int* q_start, const int* slots, int n_seqs, int heads,
                                  int group, int rows_pad, int columns, int delta, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    RecurrenceParams p{q, q_stride, k, k_stride, g, g_stride, beta, beta_stride, v, v_stride, out, out_stride, state, state_stride,
                       q_start, slots, heads, group < 1 ? 1 : group, columns};
    // Narrower CTAs while the step has fewer than two per multiprocessor: the walk is a chain of dependent steps, so its
    // time is that of one CTA, and more of them only cost reads of q, k and g that the second-level cache serves.  A
    // small step (no more than a warp per scheduler even so) puts a column over 16 lanes instead of 8: half the
    // instructions per warp and token for one more round of shuffles.  (Over 32 lanes: measured, no faster.)
    const long narrow_warps = (long)n_seqs * heads * ((columns + 3) / 4);
    const bool wide = rows_pad >= 64 && narrow_warps * 2 <= 148L * 4;
    const int rl = wide ? 16 : ROW_LANES;
    int cols_cta = wide ? 16 : COLS_PER_CTA;
    while (cols_cta > 8 && (long)n_seqs * heads * ((columns + cols_cta - 1) / cols_cta) < 2 * 148) cols_cta >>= 1;
    const dim3 grid(n_seqs * heads, (columns + cols_cta - 1) / cols_cta);
    const int threads = cols_cta * rl;
    static bool sized = false;          // once: the attribute is a property of the function, not of a launch
#define RS_REC_SIZE(RPT, RL)                                                                                                    \
    cudaFuncSetAttribute(state_recurrence_kernel<RPT, true, RL>, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                         (int)RecurrenceStage<RPT * RL>::BYTES);                                                                \
    cudaFuncSetAttribute(state_recurrence_kernel<RPT, false, RL>, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                         (int)RecurrenceStage<RPT * RL>::BYTES);
    if (!sized) {
        RS_REC_SIZE(4, 8) RS_REC_SIZE(8, 8) RS_REC_SIZE(16, 8) RS_REC_SIZE(32, 8)
        RS_REC_SIZE(4, 16) RS_REC_SIZE(8, 16) RS_REC_SIZE(16, 16)
        sized = true;
    }
#undef RS_REC_SIZE
#define RS_REC(RPT, RL)                                                                                                         \
    if (rows_pad == RPT * RL && rl == RL) {                                                                                     \
        if (delta) state_recurrence_kernel<RPT, true, RL><<<grid, threads, RecurrenceStage<RPT * RL>::BYTES, stream>>>(p);      \
        else state_recurrence_kernel<RPT, false, RL><<<grid, threads, RecurrenceStage<RPT * RL>::BYTES, stream>>>(p);           \
        return rs_launch_result();                                                                                              \
    }
    RS_REC(4, 8) RS_REC(8, 8) RS_REC(16, 8) RS_REC(32, 8) RS_REC(4, 16) RS_REC(8, 16) RS_REC(16, 16)
#undef RS_REC
    return (int)cudaErrorInvalidValue;
}

RS_EXPORT int rs_hgrn2_prep(const float* proj, long proj_stride, const void* f_bias, int fb_dt, const void* lower, int lo_dt, float* q,
                            float* g, float* w, int heads, int dim, int rows_pad, int n_tokens, cudaStream_t stream) {
    const long n = (long)n_tokens * heads * rows_pad;
    if (n <= 0) return 0;
    hgrn2_prep_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(proj, proj_stride, f_bias, fb_dt, lower, lo_dt, q, g, w, heads,
                                                                      dim, rows_pad, n);
    return rs_launch_result();
}

RS_EXPORT int rs_delta_prep(const float* proj, long proj_stride, const void* conv, int conv_dt, float* tail, long tail_stride,
                            const float* step, long step_stride, const void* dt_bias, int dtb_dt, const void* a_log, int al_dt,
                            float* q, float* k, float* g, float* v, float* beta, const int* seq_of_token, const int* q_start,
                            const int* slots, int taps, int qk_heads, int heads, int dim, int vdim, int rows_pad, int beta_off,
                            float unit_eps, float q_scale, int n_tokens, int n_seqs, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dim > 32 * MAX_PER_LANE || vdim > 32 * MAX_PER_LANE || rows_pad > 32 * MAX_PER_LANE) return (int)cudaErrorInvalidValue;
    DeltaPrepParams p{proj, proj_stride, conv, conv_dt, tail, tail_stride, step, step_stride, dt_bias, dtb_dt, a_log, al_dt,
                      q, k, g, v, beta, seq_of_token, q_start, slots, 2 * qk_heads * dim + heads * vdim, taps, qk_heads, heads,
                      dim, vdim, rows_pad, beta_off, n_tokens, unit_eps, q_scale};
    const long warps = (long)n_tokens * (2 * qk_heads + 2 * heads);
    delta_prep_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(p);
    int rc = rs_launch_result();
    if (rc || taps <= 1 || !conv) return rc;
    const long n = (long)n_seqs * p.C;
    conv_tail_update_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(proj, proj_stride, tail, tail_stride, q_start, slots,
                                                                            p.C, taps, n_seqs);
    return rs_launch_result();
}

RS_EXPORT int rs_head_norm_gate(const float* o, long o_stride, const void* weight, int w_dt, const float* gate, long gate_stride,
                                void* out, int out_dt, long out_stride, int heads, int vdim, float eps, int n_tokens,
                                int gate_silu, cudaStream_t stream) {
    const long warps = (long)n_tokens * heads;
    if (warps <= 0) return 0;
    head_norm_gate_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(o, o_stride, weight, w_dt, gate, gate_stride, out, out_dt,
                                                                          out_stride, heads, vdim, eps, n_tokens, gate_silu);
    return rs_launch_result();
}

RS_EXPORT int rs_retention_prep(const float* proj, long proj_stride, const float* cos_sin, int n_rot, int table_rows,
                                const int* positions, int pos_stride, float k_scale, float* q, float* k, int heads, int dim,
                                int rows_pad, int n_tokens, int* status, cudaStream_t stream) {
    const long n = (long)n_tokens * heads * rows_pad;
    if (n <= 0) return 0;
    if ((n_rot & 1) || n_rot > dim || (n_rot > 0 && (!cos_sin || table_rows < 1))) return (int)cudaErrorInvalidValue;
    retention_prep_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(proj, proj_stride, cos_sin, n_rot, table_rows, positions,
                                                                          pos_stride, k_scale, q, k, heads, dim, rows_pad, n, status);
    return rs_launch_result();
}

RS_EXPORT int rs_activation(const void* x, long x_stride, void* out, long out_stride, int dt, int width, int n_rows, int kind,
                            const void* pq, int pq_dt, cudaStream_t stream) {
    const long n = (long)n_rows * width;
    if (n <= 0) return 0;
    if (kind == ACT_XIELU && !pq) return (int)cudaErrorInvalidValue;
    const int esz = dt == RS_F32 ? 4 : 2, v = 16 / esz;
    if (width % v == 0 && x_stride % v == 0 && out_stride % v == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const long pieces = n / v;
        const unsigned blocks = (unsigned)((pieces + 255) / 256 < 148 * 16 ? (pieces + 255) / 256 : 148 * 16);
        RS_DISPATCH_DTYPE(dt, T, (activation_vec_kernel<T><<<blocks, 256, 0, stream>>>(
            reinterpret_cast<const T*>(x), x_stride, reinterpret_cast<T*>(out), out_stride, width, n_rows, kind, pq, pq_dt)));
        return rs_launch_result();
    }
    RS_DISPATCH_DTYPE(dt, T, (activation_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const T*>(x), x_stride, reinterpret_cast<T*>(out), out_stride, width, n, kind, pq, pq_dt)));
    return rs_launch_result();
}

RS_EXPORT int rs_scale_rows(float* x, long stride, int width, int n_rows, float scale, cudaStream_t stream) {
    const long n = (long)n_rows * width;
    if (n <= 0) return 0;
    scale_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, stride, width, n, scale);
    return rs_launch_result();
}
