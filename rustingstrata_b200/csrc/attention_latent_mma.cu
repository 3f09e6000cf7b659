// Attention over a one-plane paged cache whose rows are key and value at once (a latent shared by all query heads),
// on the warp-level tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 accumulation), for prompt portions and
// for single query tokens (split form).  The bfloat16 engine's kernel of latent attention for rows of up to 576
// values (a 512-wide latent with a 64-wide rotated part).
//
// A CTA of 8 warps owns 16 query rows: (tokens of a tile) x (query heads of a chunk), all reading the same key rows.
// Key tiles of 64 keys are streamed through two shared-memory buffers with cp.async (tile i + 1 loads under tile i), or
// through one where two would keep a second CTA off the SM.
// Per tile:
//   1. S = Q K^T: warp w computes the 16 x 8 block of keys 8w .. 8w + 7 over the whole row width, scales and masks it
//      (causal, window, the split's range) and leaves it in shared memory;
//   2. online softmax in float32: 16 threads per row take the tile's maximum, the probabilities (rounded to bfloat16
//      for the product; with split_p in two bfloat16 terms, p = hi + lo with |lo| <= 2^-9 p, both of which are multiplied,
//      so that the product carries the float32 weight), the running sum and the factor by which the row's earlier
//      results shrink;
//   3. O += P V with V the same key rows: warp w owns a slice of the row's coordinates (an eighth, rounded up to 8).
// Key tiles start at multiples of 64 from key 0 and the split form's splits at multiples of the split size, so the order
// in which a query's keys are reduced depends on its position alone.  The split form leaves un-normalised partial
// results (sum, maximum, denominator) per (sequence, split, head) that a second kernel merges in ascending order,
// the layout and order of the CUDA-core kernel (attention_simt.cu).
#include "mma_helpers.cuh"
#include <math.h>
#include <atomic>

namespace {
constexpr int KT = 64, ROWS = 16, WARPS = 8, THREADS = WARPS * 32, NT_MAX = 9, MAX_LAT = 576;
constexpr int S_PITCH = KT + 4, P_PITCH = KT + 8, MERGE_CACHED = 512;

struct LatParams {
    const __nv_bfloat16* q; long q_stride;          // [tokens, q_stride], head h at h * lat
    __nv_bfloat16* out; long out_stride;
    const __nv_bfloat16* cache; long page_stride;   // [pages][page_size][lat]
    int num_pages, page_size;
    const int* block_table; int table_stride;
    const int* q_start; const int* kv_len; const int* work;
    int n_heads, lat, hc, tok_per_cta, window;
    float scale;
    int decode, split_keys, max_splits;
    const int* split_start; float* partial; int partial_slots;
    int* status;
    int n_buf;                                      // key buffers in shared memory: 2 (tile i + 1 loads under tile i) or 1
    int split_p;                                    // 1: the softmax weights enter P V in two bfloat16 terms
};

__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// KS: k steps of 16 whose query fragments a warp keeps in registers across all key tiles (rows of up to 16 KS values);
// 0: the fragments are read from shared memory at every use (any row width).
template <int KS>
__global__ void __launch_bounds__(THREADS, 1) latent_attention_kernel(const LatParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lat = p.lat, pitch = lat + 8, chunks = lat >> 3;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [ROWS][pitch]
    __nv_bfloat16* Ks = Qs + ROWS * pitch;                                          // [n_buf][KT][pitch]
    float* Ss = reinterpret_cast<float*>(Ks + p.n_buf * KT * pitch);                      // [ROWS][S_PITCH]
    __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(Ss + ROWS * S_PITCH);      // [ROWS][P_PITCH]
    __nv_bfloat16* Pl = Ps + ROWS * P_PITCH;                                        // [ROWS][P_PITCH] the weights' second terms
    float* stat_m = reinterpret_cast<float*>(Pl + ROWS * P_PITCH);                  // [ROWS] each
    float* stat_l = stat_m + ROWS;
    float* stat_c = stat_l + ROWS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    int seq, q_off, n_q_tok;
    if (p.decode) { seq = p.work[blockIdx.x]; q_off = 0; n_q_tok = 1; }
    else { seq = p.work[2 * blockIdx.x]; q_off = p.work[2 * blockIdx.x + 1]; }
    const int row0 = p.q_start[seq];
    const int q_len = p.q_start[seq + 1] - row0;
    const int kv_len = p.kv_len[seq];
    if (!p.decode) n_q_tok = min(p.tok_per_cta, q_len - q_off);
    const int qpos0 = kv_len - q_len + q_off;
    const int head0 = blockIdx.y * p.hc;

    int key_lo = p.window > 0 ? max(0, qpos0 - p.window + 1) : 0;
    int key_hi = min(kv_len, qpos0 + n_q_tok);
    int split_local = 0;
    if (p.decode) {
        const int first_split = key_lo / p.split_keys;
        split_local = blockIdx.z;
        const int s = first_split + split_local;
        key_lo = max(key_lo, s * p.split_keys);
        key_hi = min(key_hi, (s + 1) * p.split_keys);
        if (key_lo >= key_hi) return;
    }

    // queries: row r = token (r / hc), head head0 + r % hc; rows beyond the tile's tokens or the model's heads are zero
    for (int i = tid; i < ROWS * chunks; i += THREADS) {
        const int r = i / chunks, ch = i - r * chunks;
        const int tl = r / p.hc, h = head0 + r % p.hc;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tl < n_q_tok && h < p.n_heads)
            v = *reinterpret_cast<const uint4*>(p.q + (size_t)(row0 + q_off + tl) * p.q_stride + (size_t)h * lat + ch * 8);
        *reinterpret_cast<uint4*>(Qs + r * pitch + ch * 8) = v;
    }
    if (tid < ROWS) { stat_m[tid] = -INFINITY; stat_l[tid] = 0.f; stat_c[tid] = 1.f; }

    const int* table = p.block_table + (size_t)seq * p.table_stride;
    auto load_tile = [&](int buf, int k0) {
        __nv_bfloat16* dst0 = Ks + (size_t)buf * KT * pitch;
        for (int i = tid; i < KT * chunks; i += THREADS) {
            const int j = i / chunks, ch = i - j * chunks;
            const int kpos = k0 + j;
            __nv_bfloat16* dst = dst0 + j * pitch + ch * 8;
            bool loaded = false;
            if (kpos >= key_lo && kpos < key_hi) {
                const int page = table[kpos / p.page_size];
                if (page >= 0 && page < p.num_pages) {
                    cp_async16(smem_addr(dst), p.cache + (size_t)page * p.page_stride + (size_t)(kpos % p.page_size) * lat + ch * 8);
                    loaded = true;
                } else if (ch == 0) {
                    atomicOr(p.status, RS_STATUS_BAD_PAGE);
                }
            }
            if (!loaded) *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    };

    // the slice of the row's coordinates this warp accumulates in step 3
    const int DW = ((lat + 63) >> 6) << 3;
    const int dim_lo = warp * DW;
    const int my_nt = max(0, min(DW, lat - dim_lo)) >> 3;
    float acc[NT_MAX][4];
#pragma unroll
    for (int n = 0; n < NT_MAX; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }

    const int k_first = (key_lo / KT) * KT;
    const int n_tiles = (key_hi - k_first + KT - 1) / KT;
    load_tile(0, k_first);
    cp_async_commit();
    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
    uint32_t qf[KS > 0 ? KS : 1][4];
    if (KS > 0) {
        __syncthreads();                                       // the queries are in shared memory
        const uint32_t qa = smem_addr(Qs + a_row * pitch + a_col);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            if (ks * 16 < lat) ldmatrix_x4(qa + ks * 32, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
            else qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
        }
    }
    for (int it = 0; it < n_tiles; ++it) {
        const int k0 = k_first + it * KT;
        if (p.n_buf == 2 && it + 1 < n_tiles) {
            load_tile((it + 1) & 1, k0 + KT);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            if (p.n_buf == 1 && it > 0) {                      // one buffer: the tile is fetched when the last one is done with
                load_tile(0, k0);
                cp_async_commit();
            }
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* Kt = Ks + (size_t)(p.n_buf == 2 ? (it & 1) : 0) * KT * pitch;
        // ---- 1. S = Q K^T for this warp's 8 keys
        {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t qa = smem_addr(Qs + a_row * pitch + a_col);
            const uint32_t kb = smem_addr(Kt + (warp * 8 + (lane & 7)) * pitch + 8 * ((lane >> 3) & 1));
            if (KS > 0) {
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    if (ks * 16 < lat) {
                        uint32_t b0, b1;
                        ldmatrix_x2(kb + ks * 32, b0, b1);
                        mma16816(c, qf[ks], b0, b1);
                    }
                }
            } else {
                for (int kk = 0; kk < lat; kk += 16) {
                    uint32_t a[4], b0, b1;
                    ldmatrix_x4(qa + kk * 2, a[0], a[1], a[2], a[3]);
                    ldmatrix_x2(kb + kk * 2, b0, b1);
                    mma16816(c, a, b0, b1);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = (lane >> 2) + 8 * (e >> 1), cc = warp * 8 + (lane & 3) * 2 + (e & 1);
                const int kpos = k0 + cc, qpos = qpos0 + r / p.hc;
                const bool ok = kpos >= key_lo && kpos < key_hi && kpos <= qpos && (p.window <= 0 || kpos > qpos - p.window);
                Ss[r * S_PITCH + cc] = ok ? c[e] * p.scale : -INFINITY;
            }
        }
        __syncthreads();
        // ---- 2. online softmax: 16 threads per row, 4 keys each
        {
            const int r = tid >> 4, j = tid & 15;
            const float4 s4 = *reinterpret_cast<const float4*>(Ss + r * S_PITCH + j * 4);
            float mx = fmaxf(fmaxf(s4.x, s4.y), fmaxf(s4.z, s4.w));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_old = stat_m[r];
            const float m_new = fmaxf(m_old, mx);
            float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f, corr = 1.f;
            if (m_new != -INFINITY) {
                p0 = __expf(s4.x - m_new); p1 = __expf(s4.y - m_new); p2 = __expf(s4.z - m_new); p3 = __expf(s4.w - m_new);
                corr = __expf(m_old - m_new);
            }
            float sum = (p0 + p1) + (p2 + p3);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            uint2 pk;
            pk.x = pack_bf16(p0, p1); pk.y = pack_bf16(p2, p3);
            *reinterpret_cast<uint2*>(Ps + r * P_PITCH + j * 4) = pk;
            if (p.split_p) {
                const __nv_bfloat162 h01 = *reinterpret_cast<const __nv_bfloat162*>(&pk.x);
                const __nv_bfloat162 h23 = *reinterpret_cast<const __nv_bfloat162*>(&pk.y);
                uint2 lo;
                lo.x = pack_bf16(p0 - __low2float(h01), p1 - __high2float(h01));
                lo.y = pack_bf16(p2 - __low2float(h23), p3 - __high2float(h23));
                *reinterpret_cast<uint2*>(Pl + r * P_PITCH + j * 4) = lo;
            }
            if (j == 0) { stat_m[r] = m_new; stat_l[r] = stat_l[r] * corr + sum; stat_c[r] = corr; }
        }
        __syncthreads();
        // ---- 3. O = O * corr + P V over this warp's coordinates
        if (my_nt > 0) {
            const float c0 = stat_c[lane >> 2], c1 = stat_c[(lane >> 2) + 8];
#pragma unroll
            for (int n = 0; n < NT_MAX; ++n) { acc[n][0] *= c0; acc[n][1] *= c0; acc[n][2] *= c1; acc[n][3] *= c1; }
            const uint32_t pa = smem_addr(Ps + a_row * P_PITCH + a_col);
            const uint32_t pl = smem_addr(Pl + a_row * P_PITCH + a_col);
            const uint32_t vb = smem_addr(Kt + (lane & 15) * pitch + dim_lo);
#pragma unroll
            for (int kk = 0; kk < KT; kk += 16) {
                uint32_t a[4], al[4] = {0u, 0u, 0u, 0u};
                ldmatrix_x4(pa + kk * 2, a[0], a[1], a[2], a[3]);
                if (p.split_p) ldmatrix_x4(pl + kk * 2, al[0], al[1], al[2], al[3]);
#pragma unroll
                for (int n = 0; n < NT_MAX; ++n) {
                    if (n < my_nt) {
                        uint32_t b0, b1;
                        ldmatrix_x2_trans(vb + (kk * pitch + n * 8) * 2, b0, b1);
                        mma16816(acc[n], a, b0, b1);
                        if (p.split_p) mma16816(acc[n], al, b0, b1);
                    }
                }
            }
        }
        __syncthreads();
    }

    // ---- results: row r = lane / 4 (+ 8), coordinates dim_lo + n * 8 + (lane % 4) * 2 (+ 1)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = (lane >> 2) + 8 * half;
        const int tl = r / p.hc, h = head0 + r % p.hc;
        if (tl >= n_q_tok || h >= p.n_heads) continue;
        if (p.decode) {
            const size_t slot = (size_t)p.split_start[blockIdx.x] + split_local;
            if (slot >= (size_t)p.partial_slots) {
                if ((lane & 3) == 0 && warp == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);
                continue;
            }
            float* dst = p.partial + (slot * p.n_heads + h) * (lat + 2);
#pragma unroll
            for (int n = 0; n < NT_MAX; ++n) {
                if (n < my_nt) {
                    const int d = dim_lo + n * 8 + (lane & 3) * 2;
                    dst[d] = acc[n][2 * half]; dst[d + 1] = acc[n][2 * half + 1];
                }
            }
            if (warp == 0 && (lane & 3) == 0) { dst[lat] = stat_m[r]; dst[lat + 1] = stat_l[r]; }
        } else {
            const float inv = 1.0f / stat_l[r];
            __nv_bfloat16* dst = p.out + (size_t)(row0 + q_off + tl) * p.out_stride + (size_t)h * lat;
#pragma unroll
            for (int n = 0; n < NT_MAX; ++n) {
                if (n < my_nt) {
                    const int d = dim_lo + n * 8 + (lane & 3) * 2;
                    *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(acc[n][2 * half] * inv, acc[n][2 * half + 1] * inv);
                }
            }
        }
    }
}

// out[token of seq, head, :] = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M), splits in ascending order
__global__ void latent_merge_kernel(const LatParams p) {
    const int w = blockIdx.x, h = blockIdx.y;
    const int seq = p.work[w];
    const int kv_len = p.kv_len[seq];
    const int key_lo = p.window > 0 ? max(0, kv_len - p.window) : 0;
    const int n_splits = (kv_len + p.split_keys - 1) / p.split_keys - key_lo / p.split_keys;
    const int lat = p.lat;
    if ((size_t)p.split_start[w] + n_splits > (size_t)p.partial_slots) {
        if (threadIdx.x == 0) atomicOr(p.status, RS_STATUS_BAD_PLAN);
        return;
    }
    const float* base = p.partial + ((size_t)p.split_start[w] * p.n_heads + h) * (lat + 2);
    const size_t split_stride = (size_t)p.n_heads * (lat + 2);
    // every thread takes the splits' maxima in (the loads are independent of each other), then the weights of up to
    // MERGE_CACHED splits and the denominator are kept in shared memory; a sequence with more splits recomputes them
    __shared__ float ws[MERGE_CACHED];
    __shared__ float stats[2];
    float M = -INFINITY;
#pragma unroll 4
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[s * split_stride + lat]);
    if (threadIdx.x < 32) {
        float den = 0.f;                                      // lanes take splits in turn, added lane by lane: a fixed order
        for (int s = threadIdx.x; s < n_splits; s += 32) {
            const float* ps = base + s * split_stride;
            const float e = __expf(ps[lat] - M);
            if (s < MERGE_CACHED) ws[s] = e;
            den = fmaf(ps[lat + 1], e, den);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
        if (threadIdx.x == 0) stats[0] = den;
    }
    __syncthreads();
    const float inv = 1.0f / stats[0];
    __nv_bfloat16* dst = p.out + (size_t)p.q_start[seq] * p.out_stride + (size_t)h * lat;
    for (int d = threadIdx.x; d < lat; d += blockDim.x) {
        float num = 0.f;
#pragma unroll 4
        for (int s = 0; s < n_splits; ++s) {
            const float* ps = base + s * split_stride;
            const float e = s < MERGE_CACHED ? ws[s] : __expf(ps[lat] - M);
            num = fmaf(ps[d], e, num);
        }
        dst[d] = __float2bfloat16_rn(num * inv);
    }
}

size_t latent_smem_bytes(int lat, int n_buf) {
    const int pitch = lat + 8;
    return (size_t)(ROWS + n_buf * KT) * pitch * 2 + (size_t)ROWS * S_PITCH * 4 + 2 * (size_t)ROWS * P_PITCH * 2 + 3 * ROWS * 4;
}

// Two CTAs on an SM hide more than a second key buffer does: where two buffers would leave room for one CTA only
// (rows wider than about 380 values), the kernel runs with one buffer and the other CTA's work covers the loads.
constexpr size_t HALF_SM_SMEM = 113 * 1024;

int heads_per_cta(int n_heads, int decode) {
    if (decode || n_heads >= ROWS) return ROWS;
    int hc = 1;
    while (hc < n_heads) hc <<= 1;
    return hc;
}
}  // namespace

RS_EXPORT int rs_attention_latent_supported(int n_heads, int lat, int page_size) {
    return n_heads > 0 && lat > 0 && lat % 16 == 0 && lat <= MAX_LAT && page_size > 0;
}

// Query tokens per work item of the portion form.
RS_EXPORT int rs_attention_latent_q_per_cta(int n_heads) { return ROWS / heads_per_cta(n_heads, 0); }

RS_EXPORT int rs_attention_latent_bf16(const void* q, long q_stride, void* out, long out_stride, const void* cache,
                                       long page_stride, int num_pages, int page_size, const int* block_table,
                                       int table_stride, const int* q_start, const int* kv_len, const int* work, int n_work,
                                       int n_heads, int lat, int window, float scale, int decode, int split_keys,
                                       int max_splits, const int* split_start, float* partial, int partial_slots,
                                       int split_p, int* status, void* stream) {
    if (n_work <= 0) return 0;
    if (!rs_attention_latent_supported(n_heads, lat, page_size) || q_stride % 8 || out_stride % 2 || page_stride % 8 ||
        ((size_t)q & 15) || ((size_t)cache & 15) || ((size_t)out & 3))
        return (int)cudaErrorInvalidValue;
    if (decode && (split_keys % KT || split_keys <= 0 || max_splits <= 0 || partial == nullptr || partial_slots <= 0 ||
                   split_start == nullptr))
        return (int)cudaErrorInvalidValue;
    LatParams p;
    p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.cache = (const __nv_bfloat16*)cache; p.page_stride = page_stride; p.num_pages = num_pages; p.page_size = page_size;
    p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.kv_len = kv_len; p.work = work;
    p.n_heads = n_heads; p.lat = lat; p.hc = heads_per_cta(n_heads, decode); p.tok_per_cta = decode ? 1 : ROWS / p.hc;
    p.window = window; p.scale = scale; p.decode = decode; p.split_keys = split_keys; p.max_splits = max_splits;
    p.split_start = split_start; p.partial = partial; p.partial_slots = partial_slots; p.status = status;
    p.split_p = split_p ? 1 : 0;
    p.n_buf = latent_smem_bytes(lat, 2) <= HALF_SM_SMEM ? 2 : 1;
    const size_t smem = latent_smem_bytes(lat, p.n_buf);
    static std::atomic<size_t> smem_allowed[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (smem > smem_allowed[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(latent_attention_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(latent_attention_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        size_t seen = smem_allowed[dev].load(std::memory_order_relaxed);
        while (seen < smem && !smem_allowed[dev].compare_exchange_weak(seen, smem, std::memory_order_release)) {}
    }
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_work, (n_heads + p.hc - 1) / p.hc, decode ? max_splits : 1);
    // Wider rows read the query fragments from shared memory: kept in registers (20 or 36 steps) they cost a CTA 175 to
    // 231 registers a thread, one CTA fits an SM instead of two, and the kernel got slower (593 against 431 us for 2,048
    // tokens, 8 heads, rows of 320).
    if (lat <= 128) latent_attention_kernel<8><<<grid, THREADS, smem, s>>>(p);
    else latent_attention_kernel<0><<<grid, THREADS, smem, s>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess || !decode) return (int)e;
    latent_merge_kernel<<<dim3(n_work, n_heads), 128, 0, s>>>(p);
    return rs_launch_result();
}
