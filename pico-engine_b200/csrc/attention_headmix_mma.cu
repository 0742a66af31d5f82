// The attention of attention_headmix.cu for bfloat16 on the tensor cores (mma.sync m16n8k16, operands by ldmatrix).
//
// A block takes 16 consecutive tokens of one sequence (one row tile of the MMA) and all heads, and visits the keys
// in blocks of KB = 64, 32 or 16 positions (what fits the shared memory; KB divides a cache page):
//   1. S_g = Q_g K_c(g)^T for every head g on the tensor cores (Q tile and the block's keys of all key/value heads
//      in shared memory as bfloat16, float32 accumulators);
//   2. float32 on the CUDA cores: scale, mask, and either the running maximum and sum of every (query, head) (first
//      pass over the keys) or p = exp(s - max) / denominator and the mixing w_h = sum_g mix[h, g] p_g (second pass);
//   3. O_h += W_h V_c(h) on the tensor cores.  W is float32 and the MMA takes bfloat16, so W is split into
//      hi = bf16(W) and lo = bf16(W - hi) and both are multiplied: the weights keep 16 bits of mantissa.
// With one range of keys a block runs both passes itself; with several ranges (single tokens with long contexts)
// the first pass of all ranges is a launch of its own, because the second needs the denominators over all keys.
// A block may also take only a slice of the value dimension (gridDim.z), when heads x value size has more 16x8
// accumulator tiles than its warps hold.
#include "common.cuh"

#define HX_THREADS 512
#define HX_WARPS 16
#define HX_QT 16
#define HX_PAD 8

struct HeadMixMmaArgs {
    const bf16* q; int q_stride;
    const bf16* k_pool; const bf16* v_pool;
    const int* table; int table_stride;
    const int* tok_pos; const int* tok_row;
    const int* tiles; int tile_tokens;
    int H, G, D, Dv, window; float scale;
    const float* sink; const float* mix;
    int KB, splits, dv_splits;
    float* stats; float* opart; bf16* out;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// rows [r0, r0 + n) of a [.., cols] bfloat16 matrix in global memory into shared rows of `pitch` elements; rows from
// `valid` on are zero.  16-byte copies where the row length allows.
__device__ __forceinline__ void load_rows(bf16* dst, int pitch, const bf16* src, int cols, int n, int valid) {
    if ((cols & 7) == 0) {
        const int per = cols >> 3;
        for (int e = threadIdx.x; e < n * per; e += HX_THREADS) {
            const int r = e / per, c8 = e % per;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < valid) v = *reinterpret_cast<const uint4*>(src + (size_t)r * cols + c8 * 8);
            *reinterpret_cast<uint4*>(dst + (size_t)r * pitch + c8 * 8) = v;
        }
    } else {
        for (int e = threadIdx.x; e < n * cols; e += HX_THREADS) {
            const int r = e / cols, c = e % cols;
            dst[(size_t)r * pitch + c] = r < valid ? src[(size_t)r * cols + c] : __float2bfloat16_rn(0.f);
        }
    }
}

// MODE 0: first pass only (writes stats).  1: second pass only (reads stats).  2: both passes, one range of keys.
template <int MODE, int NI, int HMAX>
__global__ void __launch_bounds__(HX_THREADS) headmix_mma_kernel(HeadMixMmaArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, G = a.G, D = a.D, Dv = a.Dv, KB = a.KB, per_kv = H / G;
    const int Dp = (D + 15) & ~15, Dvp = (Dv + 7) & ~7;
    const int qp = Dp + HX_PAD, vpitch = Dvp + HX_PAD, wp = KB + HX_PAD, pp = KB + HX_PAD;
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);                      // [H][16][qp]
    bf16* k_s = q_s + (size_t)H * HX_QT * qp;                           // [G][KB][qp]
    bf16* v_s = k_s + (size_t)G * KB * qp;                              // [G][KB][vpitch]
    bf16* wh_s = v_s + (size_t)G * KB * vpitch;                         // [H][16][wp]
    bf16* wl_s = wh_s + (size_t)H * HX_QT * wp;
    float* p_s = reinterpret_cast<float*>(wl_s + (size_t)H * HX_QT * wp);   // [H][16][pp]
    float* m_s = p_s + (size_t)H * HX_QT * pp;                          // [16][H]
    float* l_s = m_s + HX_QT * H;
    float* mix_s = l_s + HX_QT * H;                                     // [H][H]

    // the tile
    int row, t0, nq, p0;
    if (a.tiles == nullptr) { row = a.tok_row[blockIdx.x]; t0 = blockIdx.x; nq = 1; p0 = a.tok_pos[blockIdx.x]; }
    else {
        const int per = a.tile_tokens / HX_QT;
        const int* r = a.tiles + 4 * (blockIdx.x / per);
        const int off = (blockIdx.x % per) * HX_QT;
        if (off >= r[2]) return;
        row = r[0]; t0 = r[1] + off; nq = min(HX_QT, r[2] - off); p0 = r[3] + off;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, split = blockIdx.y;
    const int hi = p0 + nq;
    const int lo = (a.window > 0 && p0 - a.window + 1 > 0) ? (p0 - a.window + 1) & ~(KB - 1) : 0;
    int span = (hi - lo + a.splits - 1) / a.splits;
    span = (span + KB - 1) / KB * KB;
    const int k_begin = lo + split * span, k_end = min(hi, k_begin + span);
    const int* table = a.table + (size_t)row * a.table_stride;

    // queries: [h][i][d], zero beyond the tile's tokens and in the padding columns
    for (int e = tid; e < H * HX_QT * qp; e += HX_THREADS) {
        const int d = e % qp, i = (e / qp) % HX_QT, h = e / (qp * HX_QT);
        q_s[e] = (i < nq && d < D) ? a.q[(size_t)(t0 + i) * a.q_stride + (size_t)h * D + d] : __float2bfloat16_rn(0.f);
    }
    if (Dp != D) for (int e = tid; e < G * KB * qp; e += HX_THREADS) k_s[e] = __float2bfloat16_rn(0.f);
    if (Dvp != Dv) for (int e = tid; e < G * KB * vpitch; e += HX_THREADS) v_s[e] = __float2bfloat16_rn(0.f);
    for (int e = tid; e < HX_QT * H; e += HX_THREADS) { m_s[e] = -INFINITY; l_s[e] = 0.f; }
    if (MODE != 0 && a.mix) for (int e = tid; e < H * H; e += HX_THREADS) mix_s[e] = a.mix[e];

    // accumulator tiles of this warp: items (h, 8 value columns) of this block's slice of the value dimension
    const int nt_all = Dvp / 8, nt_per = (nt_all + a.dv_splits - 1) / a.dv_splits;
    const int nt_lo = blockIdx.z * nt_per, nt_hi = min(nt_all, nt_lo + nt_per);
    const int n_items = H * max(0, nt_hi - nt_lo), nt_cnt = max(1, nt_hi - nt_lo);
    float acc[NI][4];
#pragma unroll
    for (int r = 0; r < NI; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }

    const int n_kt = KB / 8, ntg = n_kt < 4 ? n_kt : 4, groups = n_kt / ntg;
#pragma unroll 1
    for (int pass = (MODE == 1 ? 1 : 0); pass < (MODE == 0 ? 1 : 2); ++pass) {
        __syncthreads();
        if (pass == 1) {
            // final maximum and 1 / denominator of every (query, head)
            for (int e = tid; e < HX_QT * H; e += HX_THREADS) {
                const int h = e % H;
                float M = a.sink ? a.sink[h] : -INFINITY, den = 0.f;
                if (MODE == 1) {
                    const float* st = a.stats + ((size_t)blockIdx.x * a.splits * HX_QT * H + e) * 2;
                    for (int s = 0; s < a.splits; ++s) M = fmaxf(M, st[(size_t)s * HX_QT * H * 2]);
                    for (int s = 0; s < a.splits; ++s) {
                        const float ms = st[(size_t)s * HX_QT * H * 2], ls = st[(size_t)s * HX_QT * H * 2 + 1];
                        if (ms > -INFINITY) den += ls * expf(ms - M);
                    }
                } else {
                    M = fmaxf(M, m_s[e]);
                    if (m_s[e] > -INFINITY) den = l_s[e] * expf(m_s[e] - M);
                }
                if (a.sink) den += expf(a.sink[h] - M);
                m_s[e] = M;
                l_s[e] = den > 0.f ? 1.0f / den : 0.f;
            }
            __syncthreads();
        }
#pragma unroll 1
        for (int kb = k_begin; kb < k_end; kb += KB) {
            const int page = table[kb / PE_PAGE], in_page = kb % PE_PAGE;
            const int valid = page >= 0 ? min(KB, k_end - kb) : 0;
            for (int c = 0; c < G; ++c) {
                load_rows(k_s + (size_t)c * KB * qp, qp, a.k_pool + (((size_t)max(page, 0) * G + c) * PE_PAGE + in_page) * D, D, KB, valid);
                if (pass == 1)
                    load_rows(v_s + (size_t)c * KB * vpitch, vpitch, a.v_pool + (((size_t)max(page, 0) * G + c) * PE_PAGE + in_page) * Dv, Dv, KB, valid);
            }
            __syncthreads();
            // 1. scores of every head: a unit is (head, group of up to 4 key tiles)
            for (int u = warp; u < H * groups; u += HX_WARPS) {
                const int h = u / groups, grp = u % groups;
                const bf16* qh = q_s + (size_t)h * HX_QT * qp;
                const bf16* kc = k_s + (size_t)(h / per_kv) * KB * qp;
                float s[4][4];
#pragma unroll
                for (int n = 0; n < 4; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
                for (int kk = 0; kk < Dp; kk += 16) {
                    uint32_t af[4];
                    ldsm_x4(af, qh + (size_t)(lane & 15) * qp + kk + (lane >> 4) * 8);
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        if (n < ntg) {
                            uint32_t bfr[2];
                            ldsm_x2(bfr, kc + (size_t)((grp * ntg + n) * 8 + (lane & 7)) * qp + kk + ((lane >> 3) & 1) * 8);
                            mma_bf16(s[n], af, bfr);
                        }
                    }
                }
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    if (n < ntg) {
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int i = (lane >> 2) + (r >> 1) * 8, j = (grp * ntg + n) * 8 + (lane & 3) * 2 + (r & 1);
                            const int key = kb + j, qpos = p0 + i;
                            const bool seen = i < nq && j < valid && key <= qpos && (a.window <= 0 || qpos - key < a.window);
                            float val;
                            if (pass == 0) val = seen ? s[n][r] * a.scale : -INFINITY;
                            else val = seen ? expf(s[n][r] * a.scale - m_s[i * H + h]) * l_s[i * H + h] : 0.f;
                            p_s[((size_t)h * HX_QT + i) * pp + j] = val;
                        }
                    }
                }
            }
            __syncthreads();
            if (pass == 0) {
                // 2a. a warp per (head, query): the block's maximum and sum join the running ones
                for (int pair = warp; pair < H * nq; pair += HX_WARPS) {
                    const int i = pair % nq, h = pair / nq;
                    const float* sr = p_s + ((size_t)h * HX_QT + i) * pp;
                    float bm = -INFINITY;
                    for (int j = lane; j < KB; j += 32) bm = fmaxf(bm, sr[j]);
                    bm = warp_max(bm);
                    if (bm > -INFINITY) {
                        const float m_old = m_s[i * H + h], m_new = fmaxf(m_old, bm);
                        float sum = 0.f;
                        for (int j = lane; j < KB; j += 32) sum += sr[j] > -INFINITY ? expf(sr[j] - m_new) : 0.f;
                        sum = warp_sum(sum);
                        if (lane == 0) {
                            l_s[i * H + h] = (m_old > -INFINITY ? l_s[i * H + h] * expf(m_old - m_new) : 0.f) + sum;
                            m_s[i * H + h] = m_new;
                        }
                    }
                }
                continue;                                    // (the loop's first __syncthreads orders the next block's writes)
            }
            // 2b. mixing: a thread per (query, key) holds the weights of all heads
            for (int e = tid; e < nq * KB; e += HX_THREADS) {    // (rows beyond the tile's tokens feed accumulator rows nobody stores)
                const int i = e / KB, j = e % KB;
                float pg[HMAX];
#pragma unroll
                for (int g = 0; g < HMAX; ++g) pg[g] = g < H ? p_s[((size_t)g * HX_QT + i) * pp + j] : 0.f;
                for (int h = 0; h < H; ++h) {
                    float w;
                    if (a.mix) {
                        w = 0.f;
#pragma unroll
                        for (int g = 0; g < HMAX; ++g) if (g < H) w = fmaf(mix_s[h * H + g], pg[g], w);
                    } else {
                        w = p_s[((size_t)h * HX_QT + i) * pp + j];
                    }
                    const bf16 whi = __float2bfloat16_rn(w);
                    wh_s[((size_t)h * HX_QT + i) * wp + j] = whi;
                    wl_s[((size_t)h * HX_QT + i) * wp + j] = __float2bfloat16_rn(w - __bfloat162float(whi));
                }
            }
            __syncthreads();
            // 3. O += W V: this warp's items, the A fragments loaded again only where the head changes
            for (int ks = 0; ks < KB; ks += 16) {
                uint32_t ah[4], al[4];
                int h_have = -1;
#pragma unroll
                for (int r = 0; r < NI; ++r) {
                    const int item = warp * NI + r;
                    if (item < n_items) {
                        const int h = item / nt_cnt, nt = nt_lo + item % nt_cnt;
                        if (h != h_have) {
                            ldsm_x4(ah, wh_s + ((size_t)h * HX_QT + (lane & 15)) * wp + ks + (lane >> 4) * 8);
                            ldsm_x4(al, wl_s + ((size_t)h * HX_QT + (lane & 15)) * wp + ks + (lane >> 4) * 8);
                            h_have = h;
                        }
                        uint32_t bfr[2];
                        ldsm_x2_trans(bfr, v_s + ((size_t)(h / per_kv) * KB + ks + (lane & 15)) * vpitch + nt * 8);
                        mma_bf16(acc[r], ah, bfr);
                        mma_bf16(acc[r], al, bfr);
                    }
                }
            }
            __syncthreads();                                 // the next block's keys and values overwrite what was just read
        }
    }

    if (MODE == 0) {
        float* st = a.stats + (((size_t)blockIdx.x * a.splits + split) * HX_QT * H) * 2;
        __syncthreads();
        for (int e = tid; e < HX_QT * H; e += HX_THREADS) { st[2 * e] = m_s[e]; st[2 * e + 1] = l_s[e]; }
        return;
    }
#pragma unroll
    for (int r = 0; r < NI; ++r) {
        const int item = warp * NI + r;
        if (item < n_items) {
            const int h = item / nt_cnt, nt = nt_lo + item % nt_cnt;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = (lane >> 2) + (c >> 1) * 8, d = nt * 8 + (lane & 3) * 2 + (c & 1);
                if (i < nq && d < Dv) {
                    if (a.splits == 1) a.out[((size_t)(t0 + i) * H + h) * Dv + d] = __float2bfloat16_rn(acc[r][c]);
                    else a.opart[(((size_t)blockIdx.x * a.splits + split) * HX_QT + i) * H * Dv + (size_t)h * Dv + d] = acc[r][c];
                }
            }
        }
    }
}

// The ranges' contributions summed in their order.
__global__ void headmix_mma_reduce_kernel(HeadMixMmaArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    int t0, nq;
    if (a.tiles == nullptr) { t0 = blockIdx.x; nq = 1; }
    else {
        const int per = a.tile_tokens / HX_QT;
        const int* r = a.tiles + 4 * (blockIdx.x / per);
        const int off = (blockIdx.x % per) * HX_QT;
        if (off >= r[2]) return;
        t0 = r[1] + off; nq = min(HX_QT, r[2] - off);
    }
    const int HD = a.H * a.Dv;
    for (int e = threadIdx.x; e < nq * HD; e += blockDim.x) {
        const int i = e / HD, r = e % HD;
        float s = 0.f;
        for (int sp = 0; sp < a.splits; ++sp) s += a.opart[(((size_t)blockIdx.x * a.splits + sp) * HX_QT + i) * HD + r];
        a.out[(size_t)(t0 + i) * HD + r] = __float2bfloat16_rn(s);
    }
}

static size_t hx_smem_bytes(int H, int G, int D, int Dv, int KB) {
    const size_t Dp = (D + 15) & ~15, Dvp = (Dv + 7) & ~7;
    return 2 * ((size_t)H * HX_QT * (Dp + HX_PAD) + (size_t)G * KB * (Dp + HX_PAD) + (size_t)G * KB * (Dvp + HX_PAD)
                + 2 * (size_t)H * HX_QT * (KB + HX_PAD))
           + 4 * ((size_t)H * HX_QT * (KB + HX_PAD) + 2 * (size_t)HX_QT * H + (size_t)H * H);
}

// How the tensor-core kernel would run these sizes: the key block (0: it does not take them) and into how many
// slices of the value dimension a tile is cut.
extern "C" int pe_attention_headmix_mma_plan(int H, int G, int D, int Dv, int* dv_splits) {
    if (H < 1 || H > 32 || G < 1 || H % G || D < 1 || Dv < 1 || D > 512 || Dv > 512) return 0;
    const int nt_all = ((Dv + 7) & ~7) / 8;
    int dvs = 1;
    while (H * ((nt_all + dvs - 1) / dvs) > 16 * HX_WARPS) ++dvs;
    if (dvs > nt_all) return 0;
    *dv_splits = dvs;
    for (int kb = 64; kb >= 16; kb >>= 1)
        if (hx_smem_bytes(H, G, D, Dv, kb) <= 220 * 1024) return kb;
    return 0;
}

extern "C" long long pe_attention_headmix_mma_scratch_floats(int n_tiles, int splits, int H, int Dv) {
    return (long long)n_tiles * splits * HX_QT * H * (2 + (splits > 1 ? Dv : 0));
}

template <int NI, int HMAX>
static int hx_launch(const HeadMixMmaArgs& a, int n_tiles, size_t smem, cudaStream_t s) {
    const dim3 grid(n_tiles, a.splits, a.dv_splits);
    if (a.splits == 1) {
        PE_TRY(cudaFuncSetAttribute(headmix_mma_kernel<2, NI, HMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        PE_TRY(pe_launch(headmix_mma_kernel<2, NI, HMAX>, grid, HX_THREADS, smem, s, a));
        PE_LAUNCH_CHECK();
        return 0;
    }
    PE_TRY(cudaFuncSetAttribute(headmix_mma_kernel<0, 1, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PE_TRY(cudaFuncSetAttribute(headmix_mma_kernel<1, NI, HMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    PE_TRY(pe_launch(headmix_mma_kernel<0, 1, 8>, dim3(n_tiles, a.splits, 1), HX_THREADS, smem, s, a));
    PE_LAUNCH_CHECK();
    PE_TRY(pe_launch(headmix_mma_kernel<1, NI, HMAX>, grid, HX_THREADS, smem, s, a));
    PE_LAUNCH_CHECK();
    PE_TRY(pe_launch(headmix_mma_reduce_kernel, n_tiles, 256, 0, s, a));
    PE_LAUNCH_CHECK();
    return 0;
}

extern "C" int pe_attention_headmix_mma(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                        const int* table, int table_stride, const int* tok_pos, const int* tok_row,
                                        const int* tiles, int n_runs, int tile_tokens, int T, int H, int G, int D, int Dv,
                                        int window, float scale, const float* sink, const float* mix, int splits,
                                        float* scratch, void* stream) {
    if (T <= 0) return 0;
    int dvs = 1;
    const int KB = pe_attention_headmix_mma_plan(H, G, D, Dv, &dvs);
    if (KB == 0 || splits < 1 || splits > 65535 || (tiles && (tile_tokens % HX_QT || n_runs <= 0))) return PE_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return PE_ERR_UNSUPPORTED;
    const int n_tiles = tiles ? n_runs * (tile_tokens / HX_QT) : T;
    HeadMixMmaArgs a = {(const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, table, table_stride, tok_pos, tok_row,
                        tiles, tile_tokens, H, G, D, Dv, window, scale, sink, mix, KB, splits, dvs, scratch,
                        scratch + (size_t)n_tiles * splits * HX_QT * H * 2, (bf16*)out};
    const size_t smem = hx_smem_bytes(H, G, D, Dv, KB);
    cudaStream_t s = (cudaStream_t)stream;
    const int nt_all = ((Dv + 7) & ~7) / 8;
    const int items = H * ((nt_all + dvs - 1) / dvs);
    const int ni = (items + HX_WARPS - 1) / HX_WARPS;
    if (H <= 8) return ni <= 4 ? hx_launch<4, 8>(a, n_tiles, smem, s) : hx_launch<16, 8>(a, n_tiles, smem, s);
    return ni <= 4 ? hx_launch<4, 32>(a, n_tiles, smem, s) : hx_launch<16, 32>(a, n_tiles, smem, s);
}
