// Talking-heads attention on the warp-level tensor cores, for a bfloat16 key/value cache: the serving path of the
// bfloat16 engine for portions of prompts and for single tokens alike (talking_attention.cu holds the CUDA-core form
// that the 32-bit engine and odd shapes use; both compute the same thing).
//
// A CTA takes up to QT neighbouring queries of one sequence, all heads, and a share of their key tiles.  Per tile of
// KEY_TILE keys, whose boundaries are multiples of KEY_TILE counted from the sequence's first key:
//   1. raw[g] = Q_g K_c(g)^T on mma.sync m16n8k16, a warp per head and half of the tile's keys.  The float32 queries are split into two
//      bfloat16 terms (x = hi + lo, |lo| <= 2^-9 |x|) and both are multiplied, so the score carries the float32
//      query and not its 8-bit rounding; accumulation is float32.  Scaled scores go to shared memory.
//   2. mixed[h] = sum_g talk[h, g] raw[g] on the CUDA cores in float32: a thread owns four neighbouring keys of one
//      query and eight output heads, so one 16-byte read of raw[g] feeds 32 multiply-adds; the causal and window
//      masks are applied here.
//   3. online softmax per (head, query) in float32, the running maximum and sum starting at (sink, 1); the weights,
//      split in two bfloat16 terms like the queries, times V on the tensor cores; a warp per head (two, each with half
//      of the value columns, when there are 8 heads or fewer).
// K of the next tile is fetched with cp.async while steps 2 and 3 run, V of the next tile while the next step 1 runs.
// When a tile's keys are shared out over several CTAs (few queries, many keys), each writes its unnormalised sums
// with its maximum and denominator, and talking_combine_kernel joins them; the sink is part 0's.
#include "mma_helpers.cuh"
#include <math.h>

namespace {
constexpr int KEY_TILE = 32;
constexpr int THREADS = 512;
constexpr int WARPS = THREADS / 32;
constexpr int SROW = KEY_TILE + 8;          // pitch of a query's row of scores: fragment stores and 16-byte reads without conflicts
constexpr int SMEM_LIMIT = 220 * 1024;

struct MmaParams {
    const float* q; long q_stride;            // [T, H * dk]
    const float* gate;                        // [T, H] or null
    const __nv_bfloat16* cache; long page_stride; long plane_stride; int num_pages, page_size, hdp;
    const int* block_table; int table_stride;
    const int* q_start; const int* kv_len;
    const int* work;                          // per CTA: sequence, first query, part, parts, first row of the tile's partial sums
    const float* talk; const float* sink;     // [H, H], [H]; either may be null
    void* out; int out_dt; long out_stride;   // [T, H * dv]
    float* partial; long partial_rows;        // [rows, H, dv + 2]: sums, maximum, denominator
    int H, G, dk, dv, window, chunk, QT; float scale;
    int* status;
};

struct Layout {                               // byte offsets into the dynamic shared memory
    int q_pitch, k_pitch, v_pitch, h8;
    size_t key_at, q_hi, q_lo, ks, vs, sraw, smix, tt, total;
};

__host__ __device__ inline Layout make_layout(int H, int G, int dk, int dv, int QT) {
    Layout L;
    L.q_pitch = H * dk + 8; L.k_pitch = G * dk + 8; L.v_pitch = G * dv + 8; L.h8 = (H + 7) / 8 * 8;
    size_t o = 0;
    L.key_at = o; o += 2 * KEY_TILE * sizeof(long long);
    L.q_hi = o; o += (size_t)QT * L.q_pitch * 2;
    L.q_lo = o; o += (size_t)QT * L.q_pitch * 2;
    L.ks = o; o += (size_t)KEY_TILE * L.k_pitch * 2;
    L.vs = o; o += (size_t)KEY_TILE * L.v_pitch * 2;
    L.sraw = o; o += (size_t)H * QT * SROW * 4;
    L.smix = o; o += (size_t)H * QT * SROW * 4;
    L.tt = o; o += (size_t)H * L.h8 * 4;
    L.total = o;
    return L;
}

constexpr float LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(x);
    lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

// keys of tile `k0` of sequence `s`: where each key's row of kv head 0 starts in the cache (-1: not a key of this tile)
__device__ __forceinline__ void locate_keys(const MmaParams& p, long long* key_at, int s, int k0, int k_begin, int k_end, int lane) {
    const int kpos = k0 + lane;
    long long at = -1;
    if (kpos >= k_begin && kpos < k_end) {
        const int page = p.block_table[(size_t)s * p.table_stride + kpos / p.page_size];
        if (page < 0 || page >= p.num_pages) atomicOr(p.status, RS_STATUS_BAD_PAGE);
        else at = (long long)page * p.page_stride + (long long)(kpos % p.page_size) * p.hdp;
    }
    key_at[lane] = at;
}

// rows [KEY_TILE][G * width] of one plane of the cache into shared memory, 16 bytes per copy; rows without a key are zero.
// Sixteen threads share a key's row: thread `sub` copies pieces sub, sub + 16, .. of the G * width / 8 the row has
// (piece j is piece j % (width / 8) of kv head j / (width / 8); the pair is stepped, not divided).
__device__ __forceinline__ void fetch_plane(const MmaParams& p, const long long* key_at, __nv_bfloat16* dst, int pitch, int width,
                                            size_t plane_off, int tid) {
    static_assert(THREADS == KEY_TILE * 16, "sixteen threads per key");
    const int chunks = width / 8, per_key = p.G * chunks;
    const size_t head_stride = (size_t)p.page_size * p.hdp;
    const int kk = tid >> 4, sub = tid & 15;
    const long long at = key_at[kk];
    __nv_bfloat16* row = dst + (size_t)kk * pitch;
    const __nv_bfloat16* src = p.cache + (at < 0 ? 0 : at) + plane_off;
    int c = sub / chunks, ch = sub - c * chunks;
    for (int j = sub; j < per_key; j += 16) {
        __nv_bfloat16* d = row + c * width + ch * 8;
        if (at >= 0) cp_async16(smem_addr(d), src + c * head_stride + ch * 8);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
        ch += 16;
        while (ch >= chunks) { ch -= chunks; ++c; }
    }
}

// HPW: heads a warp owns in step 3 (heads warp, warp + WARPS, ...); DVP: blocks of 16 value columns held per head
template <int HPW, int DVP>
__global__ void __launch_bounds__(THREADS, 1) talking_mma_kernel(MmaParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = p.H, G = p.G, dk = p.dk, dv = p.dv, QT = p.QT, r = p.H / p.G;
    const Layout L = make_layout(H, G, dk, dv, QT);
    long long* key_at = reinterpret_cast<long long*>(smem_raw + L.key_at);        // [2][KEY_TILE]
    __nv_bfloat16* Qhi = reinterpret_cast<__nv_bfloat16*>(smem_raw + L.q_hi);
    __nv_bfloat16* Qlo = reinterpret_cast<__nv_bfloat16*>(smem_raw + L.q_lo);
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw + L.ks);
    __nv_bfloat16* Vs = reinterpret_cast<__nv_bfloat16*>(smem_raw + L.vs);
    float* Sraw = reinterpret_cast<float*>(smem_raw + L.sraw);                     // [H][QT][SROW]
    float* Smix = reinterpret_cast<float*>(smem_raw + L.smix);                     // [H][QT][SROW]
    float* Tt = reinterpret_cast<float*>(smem_raw + L.tt);                         // [H][h8]: Tt[g][h] = talk[h][g]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int* wk = p.work + 5 * (size_t)blockIdx.x;
    const int s = wk[0], q0 = wk[1], part = wk[2], parts = wk[3], row_base = wk[4];
    const int t_first = p.q_start[s] + q0;
    const int q_len = p.q_start[s + 1] - p.q_start[s];
    const int nq = min(QT, q_len - q0);
    const int pos0 = p.kv_len[s] - q_len + q0;
    const int k_end = pos0 + nq;
    int k_begin = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    if (p.chunk > 0) k_begin = max(k_begin, pos0 / p.chunk * p.chunk);      // chunked: nothing before the first query's block
    const int kt0 = k_begin / KEY_TILE, kt1 = (k_end + KEY_TILE - 1) / KEY_TILE;
    const int per = (kt1 - kt0 + parts - 1) / parts;
    const int t_begin = kt0 + part * per, t_end = min(kt1, t_begin + per);
    const size_t plane = (size_t)p.plane_stride;
    const int qt_shift = QT == 16 ? 4 : QT == 8 ? 3 : 2;
    const uint32_t q_hi_addr = smem_addr(Qhi), q_lo_addr = smem_addr(Qlo), ks_addr = smem_addr(Ks), vs_addr = smem_addr(Vs);
    // step 3: a warp per head; with 8 heads or fewer two warps per head, each holding half of the value columns
    const bool pair = HPW == 1 && 2 * H <= WARPS;
    const int col_half = pair ? (warp & 1) : 0;

    for (int i = tid; i < QT * H * dk; i += THREADS) {
        const int qi = i / (H * dk), c = i % (H * dk);
        const float x = qi < nq ? p.q[(size_t)(t_first + qi) * p.q_stride + c] : 0.f;
        __nv_bfloat16 hi, lo;
        split_bf16(x, hi, lo);
        Qhi[(size_t)qi * L.q_pitch + c] = hi;
        Qlo[(size_t)qi * L.q_pitch + c] = lo;
    }
    for (int i = tid; i < H * L.h8; i += THREADS) {
        const int g = i / L.h8, h = i % L.h8;
        Tt[i] = h < H ? (p.talk ? p.talk[h * H + g] : (h == g ? 1.f : 0.f)) : 0.f;
    }
    float m_run[HPW][2], l_run[HPW][2], O[HPW][DVP][2][4];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = pair ? warp >> 1 : warp + WARPS * i;
        const float sk = (p.sink && h < H) ? p.sink[h] : -INFINITY;
        m_run[i][0] = m_run[i][1] = sk;
        l_run[i][0] = l_run[i][1] = (p.sink && part == 0 && tig == 0) ? 1.f : 0.f;     // summed over the four lanes of a row at the end
#pragma unroll
        for (int a = 0; a < DVP; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int c = 0; c < 4; ++c) O[i][a][b][c] = 0.f;
    }
    if (t_begin < t_end) {
        if (tid < KEY_TILE) locate_keys(p, key_at + (t_begin & 1) * KEY_TILE, s, t_begin * KEY_TILE, k_begin, k_end, lane);
        __syncthreads();
        fetch_plane(p, key_at + (t_begin & 1) * KEY_TILE, Ks, L.k_pitch, dk, 0, tid);
        cp_async_commit();
        fetch_plane(p, key_at + (t_begin & 1) * KEY_TILE, Vs, L.v_pitch, dv, plane, tid);
        cp_async_commit();
    }
    for (int t = t_begin; t < t_end; ++t) {
        const int k0 = t * KEY_TILE;
        const long long* at_now = key_at + (t & 1) * KEY_TILE;
        long long* at_next = key_at + ((t + 1) & 1) * KEY_TILE;
        cp_async_wait<1>();                                  // this tile's K has landed (its V may still be on the way)
        __syncthreads();
        // ---- 1: raw scores, a warp per head
        if (t + 1 < t_end && tid >= THREADS - KEY_TILE) locate_keys(p, at_next, s, k0 + KEY_TILE, k_begin, k_end, lane);
        for (int task = warp; task < 2 * H; task += WARPS) {
            const int g = task >> 1, half = task & 1, c = g / r;
            float acc[2][4];
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
            const int arow = (lane & 15) < QT ? (lane & 15) : 0;
            const int mi = lane >> 3;
            const int key = half * 16 + (mi >> 1) * 8 + (lane & 7);
            const uint32_t aoff = (uint32_t)(arow * L.q_pitch + g * dk + (lane >> 4) * 8) * 2u;
            uint32_t a_hi = q_hi_addr + aoff, a_lo = q_lo_addr + aoff;
            uint32_t b_at = ks_addr + (uint32_t)(key * L.k_pitch + c * dk + (mi & 1) * 8) * 2u;
            for (int ks = 0; ks < dk / 16; ++ks, a_hi += 32u, a_lo += 32u, b_at += 32u) {      // 16 coordinates = 32 bytes a step
                uint32_t ah[4], al[4], b0, b1, b2, b3;
                ldmatrix_x4(a_hi, ah[0], ah[1], ah[2], ah[3]);
                ldmatrix_x4(a_lo, al[0], al[1], al[2], al[3]);
                ldmatrix_x4(b_at, b0, b1, b2, b3);
                mma16816(acc[0], ah, b0, b1);
                mma16816(acc[0], al, b0, b1);
                mma16816(acc[1], ah, b2, b3);
                mma16816(acc[1], al, b2, b3);
            }
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
                const int col = (2 * half + nb) * 8 + 2 * tig;
                if (gid < QT)
                    *reinterpret_cast<float2*>(Sraw + ((size_t)g * QT + gid) * SROW + col) =
                        make_float2(acc[nb][0] * p.scale, acc[nb][1] * p.scale);
                if (gid + 8 < QT)
                    *reinterpret_cast<float2*>(Sraw + ((size_t)g * QT + gid + 8) * SROW + col) =
                        make_float2(acc[nb][2] * p.scale, acc[nb][3] * p.scale);
            }
        }
        __syncthreads();
        if (t + 1 < t_end) fetch_plane(p, at_next, Ks, L.k_pitch, dk, 0, tid);
        cp_async_commit();
        // ---- 2: the mix across heads and the masks
        const int items = (L.h8 / 8) * QT * 8;
        for (int i = tid; i < items; i += THREADS) {
            const int kq = i & 7, qi = (i >> 3) & (QT - 1), hc = i >> (3 + qt_shift);
            if (qi >= nq) continue;
            float acc[8][4];
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
            for (int g = 0; g < H; ++g) {
                const float4 rw = *reinterpret_cast<const float4*>(Sraw + ((size_t)g * QT + qi) * SROW + kq * 4);
                const float4 ta = *reinterpret_cast<const float4*>(Tt + g * L.h8 + hc * 8);
                const float4 tb = *reinterpret_cast<const float4*>(Tt + g * L.h8 + hc * 8 + 4);
                const float tw[8] = {ta.x, ta.y, ta.z, ta.w, tb.x, tb.y, tb.z, tb.w};
#pragma unroll
                for (int a = 0; a < 8; ++a) {
                    acc[a][0] = fmaf(tw[a], rw.x, acc[a][0]); acc[a][1] = fmaf(tw[a], rw.y, acc[a][1]);
                    acc[a][2] = fmaf(tw[a], rw.z, acc[a][2]); acc[a][3] = fmaf(tw[a], rw.w, acc[a][3]);
                }
            }
            const int qpos = pos0 + qi;
            bool seen[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int kpos = k0 + kq * 4 + b;
                seen[b] = kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window)
                          && (p.chunk <= 0 || kpos >= qpos / p.chunk * p.chunk) && at_now[kq * 4 + b] >= 0;
            }
#pragma unroll
            for (int a = 0; a < 8; ++a) {
                const int h = hc * 8 + a;
                if (h < H)
                    *reinterpret_cast<float4*>(Smix + ((size_t)h * QT + qi) * SROW + kq * 4) =
                        make_float4(seen[0] ? acc[a][0] : -INFINITY, seen[1] ? acc[a][1] : -INFINITY,
                                    seen[2] ? acc[a][2] : -INFINITY, seen[3] ? acc[a][3] : -INFINITY);
            }
        }
        cp_async_wait<1>();                                  // this tile's V has landed (the next K may still be on the way)
        __syncthreads();
        // ---- 3: online softmax and weighted values, a warp per head
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int h = pair ? warp >> 1 : warp + WARPS * i;
            if (h >= H) continue;
            float sc[4][4];
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                float2 lo2 = make_float2(-INFINITY, -INFINITY), hi2 = lo2;
                if (gid < nq) lo2 = *reinterpret_cast<const float2*>(Smix + ((size_t)h * QT + gid) * SROW + nb * 8 + 2 * tig);
                if (gid + 8 < nq) hi2 = *reinterpret_cast<const float2*>(Smix + ((size_t)h * QT + gid + 8) * SROW + nb * 8 + 2 * tig);
                sc[nb][0] = lo2.x; sc[nb][1] = lo2.y; sc[nb][2] = hi2.x; sc[nb][3] = hi2.y;
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                mx[0] = fmaxf(mx[0], fmaxf(sc[nb][0], sc[nb][1]));
                mx[1] = fmaxf(mx[1], fmaxf(sc[nb][2], sc[nb][3]));
            }
            float alpha[2], neg_m[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
                mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
                const float m_new = fmaxf(m_run[i][e], mx[e]);
                alpha[e] = m_new == -INFINITY ? 1.f : __expf(m_run[i][e] - m_new);
                m_run[i][e] = m_new;
                neg_m[e] = m_new == -INFINITY ? 0.f : -m_new * LOG2E;         // exp(s - m) = 2^(s log2 e - m log2 e); 2^-inf = 0
            }
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int nb = 0; nb < 4; ++nb)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const float v = ex2_approx(fmaf(sc[nb][b], LOG2E, neg_m[b >> 1]));
                    sc[nb][b] = v;
                    psum[b >> 1] += v;
                }
            l_run[i][0] = l_run[i][0] * alpha[0] + psum[0];
            l_run[i][1] = l_run[i][1] * alpha[1] + psum[1];
#pragma unroll
            for (int a = 0; a < DVP; ++a)
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    O[i][a][b][0] *= alpha[0]; O[i][a][b][1] *= alpha[0];
                    O[i][a][b][2] *= alpha[1]; O[i][a][b][3] *= alpha[1];
                }
            const int vcol = (h / r) * dv;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t ah[4], al[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {             // a0: row gid, keys 2 tig..; a1: row gid + 8; a2, a3: the next 8 keys
                    const float x0 = sc[2 * j + (e >> 1)][(e & 1) * 2], x1 = sc[2 * j + (e >> 1)][(e & 1) * 2 + 1];
                    const __nv_bfloat162 hh = __floats2bfloat162_rn(x0, x1);
                    const __nv_bfloat162 ll = __floats2bfloat162_rn(x0 - __low2float(hh), x1 - __high2float(hh));
                    ah[e] = *reinterpret_cast<const uint32_t*>(&hh);
                    al[e] = *reinterpret_cast<const uint32_t*>(&ll);
                }
                const uint32_t v_at = vs_addr + (uint32_t)((j * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * L.v_pitch + vcol + (lane >> 4) * 8) * 2u;
#pragma unroll
                for (int a = 0; a < DVP; ++a) {
                    if (a * 16 >= dv || (pair && (a >= DVP / 2) != (col_half == 1))) continue;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(v_at + a * 32u, b0, b1, b2, b3);
                    mma16816(O[i][a][0], ah, b0, b1);
                    mma16816(O[i][a][0], al, b0, b1);
                    mma16816(O[i][a][1], ah, b2, b3);
                    mma16816(O[i][a][1], al, b2, b3);
                }
            }
        }
        __syncthreads();
        if (t + 1 < t_end) fetch_plane(p, at_next, Vs, L.v_pitch, dv, plane, tid);
        cp_async_commit();
    }
    cp_async_wait_all();
    // ---- the end: o / l * gate, or this part's sums for the combine kernel
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = pair ? warp >> 1 : warp + WARPS * i;
        if (h >= H) continue;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            l_run[i][e] += __shfl_xor_sync(0xffffffffu, l_run[i][e], 1);
            l_run[i][e] += __shfl_xor_sync(0xffffffffu, l_run[i][e], 2);
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int qi = gid + 8 * e;
            if (qi >= nq) continue;
            if (parts == 1) {
                float f = l_run[i][e] > 0.f ? 1.0f / l_run[i][e] : 0.f;
                if (p.gate) f *= p.gate[(size_t)(t_first + qi) * H + h];
                const size_t o = (size_t)(t_first + qi) * p.out_stride + (size_t)h * dv;
#pragma unroll
                for (int a = 0; a < DVP; ++a)
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const int d = a * 16 + b * 8 + 2 * tig;
                        if (d >= dv || (pair && (a >= DVP / 2) != (col_half == 1))) continue;
                        const float y0 = O[i][a][b][2 * e] * f, y1 = O[i][a][b][2 * e + 1] * f;
                        if (p.out_dt == RS_F32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + o + d) = make_float2(y0, y1);
                        else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o + d) = __floats2bfloat162_rn(y0, y1);
                    }
            } else {
                const long row = (long)row_base + (long)part * nq + qi;
                if (row >= p.partial_rows) { if (tig == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN); continue; }
                float* dst = p.partial + ((size_t)row * H + h) * (dv + 2);
#pragma unroll
                for (int a = 0; a < DVP; ++a)
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const int d = a * 16 + b * 8 + 2 * tig;
                        if (d < dv && !(pair && (a >= DVP / 2) != (col_half == 1)))
                            *reinterpret_cast<float2*>(dst + d) = make_float2(O[i][a][b][2 * e], O[i][a][b][2 * e + 1]);
                    }
                if (tig == 0 && col_half == 0) { dst[dv] = m_run[i][e]; dst[dv + 1] = l_run[i][e]; }
            }
        }
    }
}

// joins the parts of every tile whose keys were shared out: a CTA per work item, those of part 0 do the work
__global__ void __launch_bounds__(1024) talking_combine_kernel(MmaParams p) {
    const int* wk = p.work + 5 * (size_t)blockIdx.x;
    const int s = wk[0], q0 = wk[1], part = wk[2], parts = wk[3], row_base = wk[4];
    if (part != 0 || parts <= 1) return;
    if (parts > 32) { if (threadIdx.x == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN); return; }     // a lane per part
    const int H = p.H, dv = p.dv;
    const int t_first = p.q_start[s] + q0;
    const int nq = min(p.QT, p.q_start[s + 1] - p.q_start[s] - q0);
    if ((long)row_base + (long)parts * nq > p.partial_rows) return;           // flagged by the kernel that wrote the parts
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    // a warp per (query, head): lane i holds part i's maximum and denominator, then the lanes share out the columns
    for (int rowi = warp; rowi < nq * H; rowi += warps) {
        const int qi = rowi / H, h = rowi % H;
        const size_t pitch = (size_t)nq * H * (dv + 2);                        // from one part of the row to the next
        const float* first = p.partial + ((size_t)(row_base + qi) * H + h) * (dv + 2);
        float mi = -INFINITY, li = 0.f;
        if (lane < parts) { mi = first[lane * pitch + dv]; li = first[lane * pitch + dv + 1]; }
        float m = mi;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float wi = mi == -INFINITY ? 0.f : expf(mi - m);
        float den = wi * li;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        float f = den > 0.f ? 1.0f / den : 0.f;
        if (p.gate) f *= p.gate[(size_t)(t_first + qi) * H + h];
        const size_t o0 = (size_t)(t_first + qi) * p.out_stride + (size_t)h * dv;
        for (int d0 = 0; d0 < dv; d0 += 64) {                                   // every lane walks every round: the shuffles need them
            const int d = d0 + 2 * lane;
            float y0 = 0.f, y1 = 0.f;
            for (int pt = 0; pt < parts; ++pt) {
                const float w = __shfl_sync(0xffffffffu, wi, pt);
                if (d < dv) {
                    const float2 x = *reinterpret_cast<const float2*>(first + pt * pitch + d);
                    y0 = fmaf(w, x.x, y0); y1 = fmaf(w, x.y, y1);
                }
            }
            if (d >= dv) continue;
            y0 *= f; y1 *= f;
            if (p.out_dt == RS_F32) *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + o0 + d) = make_float2(y0, y1);
            else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o0 + d) = __floats2bfloat162_rn(y0, y1);
        }
    }
}

bool shape_ok(int H, int G, int dk, int dv) {
    if (H < 1 || G < 1 || H % G || dk % 16 || dv % 16 || dk < 16 || dv < 16) return false;
    const int hpw = (H + WARPS - 1) / WARPS;
    return (hpw == 1 && dv <= 128) || (hpw == 2 && dv <= 64);
}

template <int HPW, int DVP>
int launch(const MmaParams& p, int n_work, size_t smem, cudaStream_t stream) {
    static bool sized = false;          // once: the attribute is a property of the function, not of a launch
    if (!sized) {
        cudaFuncSetAttribute(talking_mma_kernel<HPW, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        sized = true;
    }
    talking_mma_kernel<HPW, DVP><<<n_work, THREADS, smem, stream>>>(p);
    return rs_launch_result();
}
}  // namespace

// the largest number of queries a CTA of the tensor-core form can take (0: the shape is not one of its shapes)
RS_EXPORT int rs_talking_attention_mma_q_per_cta(int H, int G, int dk, int dv) {
    if (!shape_ok(H, G, dk, dv)) return 0;
    for (int qt = 16; qt >= 4; qt >>= 1)
        if (make_layout(H, G, dk, dv, qt).total <= SMEM_LIMIT) return qt;
    return 0;
}

// work: n_work rows of (sequence, first query, part, parts, first row of the tile's partial sums); any_parts: some
// row has parts > 1 (the combine kernel runs)
RS_EXPORT int rs_talking_attention_mma(const float* q, long q_stride, const float* gate, const void* cache, long page_stride,
                                       int num_pages, int page_size, int hdp, const int* block_table, int table_stride,
                                       const int* q_start, const int* kv_len, const int* work, int n_work, int any_parts,
                                       const float* talk, const float* sink, void* out, int out_dt, long out_stride,
                                       float* partial, long partial_rows, int H, int G, int dk, int dv, int window, int chunk,
                                       int QT, float scale, int* status, cudaStream_t stream) {
    if (n_work <= 0) return 0;
    if (!shape_ok(H, G, dk, dv) || (QT != 4 && QT != 8 && QT != 16) || hdp % 8 || (any_parts && !partial))
        return (int)cudaErrorInvalidValue;
    const size_t smem = make_layout(H, G, dk, dv, QT).total;
    if (smem > SMEM_LIMIT) return (int)cudaErrorInvalidValue;
    MmaParams p{q, q_stride, gate, reinterpret_cast<const __nv_bfloat16*>(cache), page_stride, (long)G * page_size * hdp, num_pages,
                page_size, hdp, block_table, table_stride, q_start, kv_len, work, talk, sink, out, out_dt, out_stride, partial,
                partial_rows, H, G, dk, dv, window, chunk, QT, scale, status};
    int rc;
    if (H > WARPS) rc = launch<2, 4>(p, n_work, smem, stream);
    else if (dv <= 64) rc = launch<1, 4>(p, n_work, smem, stream);
    else rc = launch<1, 8>(p, n_work, smem, stream);
    if (rc) return rc;
    if (any_parts) {
        // a warp's rows are chains of dependent loads: many warps, few rows each
        talking_combine_kernel<<<n_work, QT * H >= 64 ? 1024 : 256, 0, stream>>>(p);
        return rs_launch_result();
    }
    return 0;
}
