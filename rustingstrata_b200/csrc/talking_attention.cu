// Attention whose scores are mixed across heads before the softmax ("talking heads"), with a learned sink in every
// head's denominator and a gate per head on the way out, over the paged key/value cache, for both engines:
//   * talking_attention_prep: biases, RMS norm of every q and k head (or one norm over the whole q row and one over the
//     whole k row, with a weight per coordinate), rotation of neighbouring pairs or of the halves of the rotated prefix,
//     q to float32 rows, k and v into the request's cache pages, sigmoid of the head gates;
//   * talking_attention: for a tile of queries of one sequence, key tile by key tile: raw scores of all heads,
//     mixed[h] = sum_g talk[h, g] raw[g], online softmax per (head, query) whose running maximum and sum start at
//     (sink, 1) instead of (-inf, 0), weighted sum of values, and at the end o / l * gate.
// A query sees the keys up to its own position, within ``window`` keys if there is a window, and within its own block
// of ``chunk`` positions (counted from the sequence's first) if the attention is chunked.
// Scores, weights, the mix and the sums are float32; keys and values have the cache's element type.  Key tiles start
// at multiples of KEY_TILE counted from the sequence's first key, so the order in which a query's keys enter its sums
// does not depend on how the sequence was cut into steps or on what else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int MAX_PER_LANE = 8;          // heads of up to 256 channels
constexpr int KEY_TILE = 32;
constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
constexpr int SMEM_LIMIT = 200 * 1024;     // dynamic shared memory a CTA of the attention kernel may ask for

__device__ __forceinline__ void store_any(void* p, int dt, size_t i, float v) {
    if (dt == RS_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

struct PrepParams {
    const float* proj; long proj_stride;      // [T, q (H * dk) | k (G * dk) | v (G * dv) | gate (H)]
    const void* bias; int bias_dt;            // [H * dk + G * dk + G * dv] or null
    const void* q_norm; const void* k_norm; int norm_dt; float eps;     // [dk] each, or null: no norm
    int row_norm;                             // 1: one norm over the whole q row and one over the whole k row, weights [H * dk], [G * dk]
    const float* cos_sin; int n_rot; int table_rows;                     // [rows, cos(n_rot / 2) | sin(n_rot / 2)]
    int half_pairs;                           // 0: coordinate 2i turns with 2i + 1; 1: coordinate i with i + n_rot / 2
    float* q_out; long q_stride;              // [T, H * dk]
    float* gate_out;                          // [T, H] or null
    void* cache; int cache_dt; long page_stride; long plane_stride; int num_pages, page_size, hdp;
    const int* block_table; int table_stride;
    const int* positions; int pos_stride; const int* seq_of_token;
    int H, G, dk, dv, n_tokens, write_kv, has_gate;
    int* status;
};

// One (token, item): the q heads, then the k heads, then the v heads, then one item for the gates.  ``inv_q`` and
// ``inv_k`` are the row norms' factors (row_norm only); ``turn`` is the warp's 256 floats of shared memory.
__device__ __forceinline__ void prep_item(const PrepParams& p, int t, int item, int lane, float inv_q, float inv_k, float* turn) {
    const int kv_items = p.write_kv ? 2 * p.G : 0;
    const float* row = p.proj + (size_t)t * p.proj_stride;
    if (item == p.H + kv_items) {
        const int off = p.H * p.dk + p.G * (p.dk + p.dv);
        for (int h = lane; h < p.H; h += 32) p.gate_out[(size_t)t * p.H + h] = 1.0f / (1.0f + expf(-row[off + h]));
        return;
    }
    int kind, head, base, width;
    if (item < p.H) { kind = 0; head = item; base = head * p.dk; width = p.dk; }
    else if (item < p.H + p.G) { kind = 1; head = item - p.H; base = (p.H + head) * p.dk; width = p.dk; }
    else { kind = 2; head = item - p.H - p.G; base = (p.H + p.G) * p.dk + head * p.dv; width = p.dv; }
    const int pos = p.positions[(size_t)t * p.pos_stride];
    float x[MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int m = 0; m < MAX_PER_LANE; ++m) {
        const int d = lane + 32 * m;
        x[m] = 0.f;
        if (d < width) {
            x[m] = row[base + d] + (p.bias ? load_any(p.bias, p.bias_dt, base + d) : 0.f);
            ss = fmaf(x[m], x[m], ss);
        }
    }
    if (kind != 2) {
        const void* nw = kind == 0 ? p.q_norm : p.k_norm;
        if (nw) {
            float r;
            int w0 = 0;
            if (p.row_norm) {
                r = kind == 0 ? inv_q : inv_k;
                w0 = head * p.dk;                    // the weight has a value per coordinate of the row
            } else {
                ss = warp_sum(ss);
                r = 1.0f / sqrtf(ss / (float)width + p.eps);
            }
#pragma unroll
            for (int m = 0; m < MAX_PER_LANE; ++m) {
                const int d = lane + 32 * m;
                if (d < width) x[m] = x[m] * r * load_any(nw, p.norm_dt, w0 + d);
            }
        }
        if (p.n_rot > 0) {
            const int half = p.n_rot >> 1;
            const int trow = pos < p.table_rows ? pos : p.table_rows - 1;
            if (pos >= p.table_rows && lane == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);       // a position the table does not hold
            const float* cs = p.cos_sin + (size_t)trow * p.n_rot;
            if (p.half_pairs) {
                // coordinate i turns with i + half: the partner lies in another lane and register, so the row makes a
                // round trip through the warp's shared memory
                __syncwarp();
#pragma unroll
                for (int m = 0; m < MAX_PER_LANE; ++m) { const int d = lane + 32 * m; if (d < p.n_rot) turn[d] = x[m]; }
                __syncwarp();
#pragma unroll
                for (int m = 0; m < MAX_PER_LANE; ++m) {
                    const int d = lane + 32 * m;
                    if (d < p.n_rot && d < width) {
                        const int i = d < half ? d : d - half;
                        const float c = cs[i], sn = cs[half + i];
                        const float other = turn[d < half ? d + half : d - half];
                        x[m] = d < half ? fmaf(x[m], c, -other * sn) : fmaf(x[m], c, other * sn);
                    }
                }
            } else {
#pragma unroll
                for (int m = 0; m < MAX_PER_LANE; ++m) {
                    const int d = lane + 32 * m;
                    const float other = __shfl_xor_sync(0xffffffffu, x[m], 1);    // coordinate d ^ 1: the pair's other half
                    if (d < p.n_rot && d < width) {
                        const float c = cs[d >> 1], sn = cs[half + (d >> 1)];
                        x[m] = (d & 1) ? fmaf(x[m], c, other * sn) : fmaf(x[m], c, -other * sn);
                    }
                }
            }
        }
    }
    if (kind == 0) {
        float* dst = p.q_out + (size_t)t * p.q_stride + (size_t)head * p.dk;
#pragma unroll
        for (int m = 0; m < MAX_PER_LANE; ++m) { const int d = lane + 32 * m; if (d < width) dst[d] = x[m]; }
        return;
    }
    const int s = p.seq_of_token[t];
    const int page = p.block_table[(size_t)s * p.table_stride + pos / p.page_size];
    if (page < 0 || page >= p.num_pages) { if (lane == 0) atomicOr(p.status, RS_STATUS_BAD_PAGE); return; }
    const size_t o = (size_t)page * p.page_stride + (kind == 2 ? p.plane_stride : 0)
                   + ((size_t)head * p.page_size + pos % p.page_size) * p.hdp;
#pragma unroll
    for (int m = 0; m < MAX_PER_LANE; ++m) {
        const int d = lane + 32 * m;
        if (d < p.hdp) store_any(p.cache, p.cache_dt, o + d, d < width ? x[m] : 0.f);
    }
}

// A warp per (token, item).
__global__ void __launch_bounds__(THREADS) talking_prep_kernel(PrepParams p) {
    __shared__ float turn[WARPS][32 * MAX_PER_LANE];
    const int items = p.H + (p.write_kv ? 2 * p.G : 0) + (p.has_gate ? 1 : 0);
    const long wid = (long)blockIdx.x * WARPS + (threadIdx.x >> 5);
    if (wid >= (long)p.n_tokens * items) return;
    prep_item(p, (int)(wid / items), (int)(wid % items), threadIdx.x & 31, 0.f, 0.f, turn[threadIdx.x >> 5]);
}

// A CTA per token for the norm over whole rows: the sums of squares of the biased q row and k row first, each thread's
// share in a fixed order and the warps' shares added in warp order, then the token's items dealt to the warps.
__global__ void __launch_bounds__(THREADS) talking_prep_rows_kernel(PrepParams p) {
    __shared__ float turn[WARPS][32 * MAX_PER_LANE];
    __shared__ float part[2][WARPS];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = p.proj + (size_t)t * p.proj_stride;
    const int nq = p.H * p.dk, nk = p.G * p.dk;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += THREADS) {
        const float v = row[i] + (p.bias ? load_any(p.bias, p.bias_dt, i) : 0.f);
        sq = fmaf(v, v, sq);
    }
    for (int i = threadIdx.x; i < nk; i += THREADS) {
        const float v = row[nq + i] + (p.bias ? load_any(p.bias, p.bias_dt, nq + i) : 0.f);
        sk = fmaf(v, v, sk);
    }
    sq = warp_sum(sq); sk = warp_sum(sk);
    if (lane == 0) { part[0][warp] = sq; part[1][warp] = sk; }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) { tq += part[0][w]; tk += part[1][w]; }
    const float inv_q = 1.0f / sqrtf(tq / (float)nq + p.eps), inv_k = 1.0f / sqrtf(tk / (float)nk + p.eps);
    const int items = p.H + (p.write_kv ? 2 * p.G : 0) + (p.has_gate ? 1 : 0);
    for (int item = warp; item < items; item += WARPS) prep_item(p, t, item, lane, inv_q, inv_k, turn[warp]);
}

struct AttnParams {
    const float* q; long q_stride;            // [T, H * dk]
    const float* gate;                        // [T, H] or null
    const void* cache; long page_stride; long plane_stride; int num_pages, page_size, hdp;
    const int* block_table; int table_stride;
    const int* q_start; const int* kv_len; const int* work;     // work: (sequence, first query of the tile) pairs
    const float* talk; const float* sink;     // [H, H], [H]; either may be null
    void* out; int out_dt; long out_stride;   // [T, H * dv]
    int H, G, dk, dv, window, chunk, QT; float scale;
    int* status;
};

template <typename T>
__global__ void __launch_bounds__(THREADS) talking_attention_kernel(AttnParams p) {
    extern __shared__ __align__(16) float smem[];
    const int H = p.H, QT = p.QT, dk = p.dk, dv = p.dv, r = p.H / p.G;
    long long* key_at = reinterpret_cast<long long*>(smem);    // [KEY_TILE] element offset of the key's row of head 0, -1: none
    float* Ks = smem + 2 * KEY_TILE;                    // [KEY_TILE][dk + 1]
    float* Sraw = Ks + KEY_TILE * (dk + 1);             // [H][QT][KEY_TILE]
    float* Smix = Sraw + H * QT * KEY_TILE;             // [H][QT][KEY_TILE]
    float* O = Smix + H * QT * KEY_TILE;                // [H * QT][dv]
    float* M = O + H * QT * dv;                         // [H * QT] running maximum
    float* L = M + H * QT;                              // [H * QT] running sum
    float* Tm = L + H * QT;                             // [H][H]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int s = p.work[2 * blockIdx.x], q0 = p.work[2 * blockIdx.x + 1];
    const int t_first = p.q_start[s] + q0;
    const int q_len = p.q_start[s + 1] - p.q_start[s];
    const int nq = min(QT, q_len - q0);
    const int pos0 = p.kv_len[s] - q_len + q0;          // position of the tile's first query
    const int k_end = pos0 + nq;                        // keys [k_begin, k_end) are seen by some query of the tile
    int k_begin = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    if (p.chunk > 0) k_begin = max(k_begin, pos0 / p.chunk * p.chunk);       // the first query's block starts no later than the others'
    const T* cache = reinterpret_cast<const T*>(p.cache);
    const size_t head_stride = (size_t)p.page_size * p.hdp;

    for (int i = tid; i < H * QT; i += THREADS) {
        const int h = i / QT;
        M[i] = p.sink ? p.sink[h] : -INFINITY;
        L[i] = p.sink ? 1.0f : 0.0f;
    }
    for (int i = tid; i < H * QT * dv; i += THREADS) O[i] = 0.f;
    if (p.talk) for (int i = tid; i < H * H; i += THREADS) Tm[i] = p.talk[i];

    for (int k0 = (k_begin / KEY_TILE) * KEY_TILE; k0 < k_end; k0 += KEY_TILE) {
        __syncthreads();                                 // the tile before this one is done with key_at, Ks and the scores
        if (tid < KEY_TILE) {
            const int kpos = k0 + tid;
            long long at = -1;
            if (kpos >= k_begin && kpos < k_end) {
                const int page = p.block_table[(size_t)s * p.table_stride + kpos / p.page_size];
                if (page < 0 || page >= p.num_pages) atomicOr(p.status, RS_STATUS_BAD_PAGE);
                else at = (long long)page * p.page_stride + (long long)(kpos % p.page_size) * p.hdp;
            }
            key_at[tid] = at;
        }
        // ---- raw scores of every head: one kv head's keys at a time through shared memory
        for (int c = 0; c < p.G; ++c) {
            __syncthreads();
            for (int i = tid; i < KEY_TILE * dk; i += THREADS) {
                const int kk = i / dk, d = i % dk;
                const long long at = key_at[kk];
                Ks[kk * (dk + 1) + d] = at < 0 ? 0.f : to_f32<T>(cache[at + (size_t)c * head_stride + d]);
            }
            __syncthreads();
            const float* krow = Ks + lane * (dk + 1);
            // the warp's (query, head of this group) pairs, four at a time; the lane is the key
            const int pairs = ((nq - warp + WARPS - 1) / WARPS) * r;
            for (int pi = 0; pi < pairs; pi += 4) {
                const float* qp[4];
                int so[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int pj = min(pi + u, pairs - 1);
                    const int qi = warp + WARPS * (pj / r), g = c * r + pj % r;
                    qp[u] = p.q + (size_t)(t_first + qi) * p.q_stride + (size_t)g * dk;
                    so[u] = (g * QT + qi) * KEY_TILE + lane;
                }
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                for (int d = 0; d < dk; ++d) {
                    const float kd = krow[d];
                    a0 = fmaf(qp[0][d], kd, a0); a1 = fmaf(qp[1][d], kd, a1);
                    a2 = fmaf(qp[2][d], kd, a2); a3 = fmaf(qp[3][d], kd, a3);
                }
                Sraw[so[0]] = a0 * p.scale;
                if (pi + 1 < pairs) Sraw[so[1]] = a1 * p.scale;
                if (pi + 2 < pairs) Sraw[so[2]] = a2 * p.scale;
                if (pi + 3 < pairs) Sraw[so[3]] = a3 * p.scale;
            }
        }
        __syncthreads();
        // ---- mix across heads, and mask what the query does not see
        for (int i = tid; i < H * nq * KEY_TILE; i += THREADS) {
            const int kk = i % KEY_TILE, qi = (i / KEY_TILE) % nq, h = i / (KEY_TILE * nq);
            const int kpos = k0 + kk, qpos = pos0 + qi;
            float v = -INFINITY;
            if (kpos <= qpos && kpos >= k_begin && (p.window <= 0 || kpos > qpos - p.window)
                && (p.chunk <= 0 || kpos >= qpos / p.chunk * p.chunk) && key_at[kk] >= 0) {
                if (p.talk) {
                    v = 0.f;
                    for (int g = 0; g < H; ++g) v = fmaf(Tm[h * H + g], Sraw[(g * QT + qi) * KEY_TILE + kk], v);
                } else {
                    v = Sraw[(h * QT + qi) * KEY_TILE + kk];
                }
            }
            Smix[(h * QT + qi) * KEY_TILE + kk] = v;
        }
        __syncthreads();
        // ---- online softmax and weighted values: a warp per (head, query) row
        const int nk = min(KEY_TILE, k_end - k0);
        for (int row = warp; row < H * nq; row += WARPS) {
            const int h = row / nq, qi = row % nq;
            const int ri = h * QT + qi;
            const float sc = Smix[ri * KEY_TILE + lane];
            const float m_old = M[ri];
            const float m_new = fmaxf(m_old, warp_max(sc));
            if (m_new == -INFINITY) continue;            // nothing seen yet and no sink
            const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            const float pr = sc == -INFINITY ? 0.f : expf(sc - m_new);
            const float psum = warp_sum(pr);
            __syncwarp();
            Smix[ri * KEY_TILE + lane] = pr;
            if (lane == 0) { M[ri] = m_new; L[ri] = L[ri] * alpha + psum; }
            __syncwarp();
            const size_t v_off = p.plane_stride + (size_t)(h / r) * head_stride;
            for (int d = lane; d < dv; d += 32) {
                float acc = O[ri * dv + d] * alpha;
                for (int kk = 0; kk < nk; ++kk) {
                    const float w = Smix[ri * KEY_TILE + kk];
                    if (w != 0.f) acc = fmaf(w, to_f32<T>(cache[key_at[kk] + v_off + d]), acc);
                }
                O[ri * dv + d] = acc;
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < H * nq * dv; i += THREADS) {
        const int d = i % dv, h = (i / dv) % H, qi = i / (dv * H);
        const int ri = h * QT + qi;
        const float l = L[ri];
        float y = l > 0.f ? O[ri * dv + d] / l : 0.f;
        if (p.gate) y *= p.gate[(size_t)(t_first + qi) * H + h];
        store_any(p.out, p.out_dt, (size_t)(t_first + qi) * p.out_stride + (size_t)h * dv + d, y);
    }
}

size_t attn_smem_bytes(int H, int QT, int dk, int dv) {
    size_t f = (size_t)KEY_TILE * (dk + 1) + 2ull * H * QT * KEY_TILE + (size_t)H * QT * dv + 2ull * H * QT + (size_t)H * H;
    return f * sizeof(float) + KEY_TILE * sizeof(long long);
}
}  // namespace

// the largest number of queries a CTA can take for these head counts and sizes (0: the shape does not fit at all)
RS_EXPORT int rs_talking_attention_q_per_cta(int H, int dk, int dv) {
    for (int qt = 16; qt >= 1; qt >>= 1)
        if (attn_smem_bytes(H, qt, dk, dv) <= SMEM_LIMIT) return qt;
    return 0;
}

RS_EXPORT int rs_talking_attention_prep(const float* proj, long proj_stride, const void* bias, int bias_dt, const void* q_norm,
                                        const void* k_norm, int norm_dt, float eps, int row_norm, const float* cos_sin, int n_rot,
                                        int table_rows, int half_pairs, float* q_out, long q_stride, float* gate_out, void* cache, int cache_dt, long page_stride,
                                        int num_pages, int page_size, int hdp, const int* block_table, int table_stride,
                                        const int* positions, int pos_stride, const int* seq_of_token, int H, int G, int dk, int dv,
                                        int n_tokens, int write_kv, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dk > 32 * MAX_PER_LANE || dv > 32 * MAX_PER_LANE || hdp > 32 * MAX_PER_LANE || (n_rot & 1) || n_rot > dk)
        return (int)cudaErrorInvalidValue;
    PrepParams p{proj, proj_stride, bias, bias_dt, q_norm, k_norm, norm_dt, eps, row_norm, cos_sin, n_rot, table_rows, half_pairs, q_out, q_stride, gate_out,
                 cache, cache_dt, page_stride, (long)G * page_size * hdp, num_pages, page_size, hdp, block_table, table_stride,
                 positions, pos_stride, seq_of_token, H, G, dk, dv, n_tokens, write_kv, gate_out != nullptr, status};
    const long warps = (long)n_tokens * (H + (write_kv ? 2 * G : 0) + (gate_out ? 1 : 0));
    if (row_norm && q_norm) talking_prep_rows_kernel<<<(unsigned)n_tokens, THREADS, 0, stream>>>(p);
    else talking_prep_kernel<<<(unsigned)((warps + WARPS - 1) / WARPS), THREADS, 0, stream>>>(p);
    return rs_launch_result();
}

RS_EXPORT int rs_talking_attention(const float* q, long q_stride, const float* gate, const void* cache, int cache_dt, long page_stride,
                                   int num_pages, int page_size, int hdp, const int* block_table, int table_stride,
                                   const int* q_start, const int* kv_len, const int* work, int n_work, const float* talk,
                                   const float* sink, void* out, int out_dt, long out_stride, int H, int G, int dk, int dv,
                                   int window, int chunk, int QT, float scale, int* status, cudaStream_t stream) {
    if (n_work <= 0) return 0;
    const size_t smem = attn_smem_bytes(H, QT, dk, dv);
    if (QT < 1 || smem > SMEM_LIMIT || H % G) return (int)cudaErrorInvalidValue;
    AttnParams p{q, q_stride, gate, cache, page_stride, (long)G * page_size * hdp, num_pages, page_size, hdp, block_table, table_stride,
                 q_start, kv_len, work, talk, sink, out, out_dt, out_stride, H, G, dk, dv, window, chunk, QT, scale, status};
    static bool sized = false;          // once: the attribute is a property of the function, not of a launch
    if (!sized) {
        cudaFuncSetAttribute(talking_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        cudaFuncSetAttribute(talking_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        sized = true;
    }
    if (cache_dt == RS_F32) {
        talking_attention_kernel<float><<<n_work, THREADS, smem, stream>>>(p);
    } else if (cache_dt == RS_BF16) {
        talking_attention_kernel<__nv_bfloat16><<<n_work, THREADS, smem, stream>>>(p);
    } else {
        return (int)cudaErrorInvalidValue;
    }
    return rs_launch_result();
}
