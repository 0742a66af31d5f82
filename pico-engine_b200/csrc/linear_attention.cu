// Linear attention with a decaying matrix state, on the projections of a step's packed tokens.
//
//   per head:   S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t        S [D, Dv], float32
//
// a_t is either one constant per head (`head_decay` [H]) or one number per key channel and token,
// a = sigmoid(z)^(inv_tau) = exp(-softplus(-z) * inv_tau) from float32 logits `z` [T, H*D].  q, k and v are columns of
// `proj` [T, ld] (heads side by side, q_off / k_off / v_off the first column of each); an activation (0: none,
// 1: silu) is applied to q and k and to v while they are loaded, and q is multiplied by `q_scale`.  Everything
// after the load is float32; o [T, H*Dv] is written as float32.  A sequence's S lives in its slot of the state
// area (`state` points at element 0 of slot 0, slots `state_stride` floats apart, [H, D, Dv] row-major) and is
// zero for a new sequence.
//
// A block owns 32 (or 64) columns of one head's S: thread (ds, j) keeps R consecutive rows of column j (and of j + 32) in registers,
// so the state is read and written with coalesced accesses and never leaves the registers in between.  Tokens
// are taken in groups of LA_GROUP: the group's q, k, a and v go to shared memory (vector reads from there), every
// thread walks the group's tokens, and the LA_DS partial sums of an output are added after the group.
//
// Two ways to run a step, equal up to float32 rounding:
//  * sequential (steps of about one token a sequence): block (sequence, head, column tile) walks the
//    sequence's tokens from the stored state and stores the new state.
//  * chunked (prompts): a sequence's tokens are cut into chunks of LA_CHUNK.  The recurrence is linear in S,
//    S_end = diag(A) S_in + L with A the product of the chunk's decays and L the chunk's own contribution, so
//    pass 1 computes (A, L) of every chunk from S_in = 0, pass 2 walks a sequence's chunks in order (an element
//    a thread), leaves each chunk's S_in where its L was and stores the sequence's new state, and pass 3 runs
//    every chunk again from its S_in and writes the outputs.  Chunks never cross sequences: chunk c of the step
//    is found from the rows' lengths on the device, so the grid depends on (T, B) only.
#include "common.cuh"

#define LA_COLS 32
#define LA_DS 8
#define LA_THREADS (LA_COLS * LA_DS)
#define LA_GROUP 8
#define LA_CHUNK 64

struct LAArgs {
    const void* proj; int ld, q_off, k_off, v_off;
    const void* z; int z_ld;
    const float* head_decay;
    float inv_tau, q_scale;
    int act_qk, act_v;
    float* state; long long state_stride;
    const int* row_first; const int* row_lens; const int* slots;
    float* out;
    int B, H, D, Dv;
    float* chunk_state;      // [chunks, H, D, Dv]
    float* chunk_decay;      // [chunks, H, D]
    int max_chunks;
};

// silu of a projection.  FAST (the bfloat16 engine, whose projections carry 8 bits): 2^x and the reciprocal from the
// special-function unit, relative error about 2^-22; else the exact routines.  A block applies it to every q and k entry of
// its head for each of its tokens, so its cost is paid once per 32 columns of the state.
template <bool FAST>
__device__ __forceinline__ float la_act(float v, int act) {
    if (act != 1) return v;
    if (FAST) {
        float e, r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * v));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
        return v * r;
    }
    return v / (1.0f + expf(-v));
}

// a = sigmoid(z)^(inv_tau), through the logarithm: -softplus(-z) * inv_tau
__device__ __forceinline__ float la_channel_decay(float z, float inv_tau) {
    const float u = -z;
    const float sp = fmaxf(u, 0.f) + log1pf(expf(-fabsf(u)));
    return expf(-sp * inv_tau);
}

// Which sequence chunk `c` of the step belongs to, its first packed token and its number of tokens (0: no such chunk).
__device__ __forceinline__ void la_find_chunk(const int* row_first, const int* row_lens, int B, int c, int& row, int& first, int& count) {
    int base = 0;
    row = -1; first = 0; count = 0;
    for (int b = 0; b < B; ++b) {
        const int n = row_lens[b], nc = (n + LA_CHUNK - 1) / LA_CHUNK;
        if (c < base + nc) {
            const int local = c - base;
            row = b; first = row_first[b] + local * LA_CHUNK;
            count = min(LA_CHUNK, n - local * LA_CHUNK);
            return;
        }
        base += nc;
    }
}

// MODE 0: a sequence's tokens from its stored state; 1: a chunk from zero, leaving (A, L); 2: a chunk from its S_in.
// NC: columns of the state a thread keeps (j and j + 32): with two, a block owns 64 columns, and every q, k and decay entry read
// from shared memory meets two columns' multiply-adds.
template <typename T, typename TZ, int R, int NC, bool PER_CHANNEL, int MODE>
__global__ void __launch_bounds__(LA_THREADS) la_walk_kernel(LAArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int DP = R * LA_DS;                       // rows the block's threads cover (D rounded up)
    constexpr int COLS = LA_COLS * NC;                  // columns the block owns
    constexpr bool FAST = sizeof(T) == 2;
    __shared__ __align__(16) float sq[LA_GROUP][DP];
    __shared__ __align__(16) float sk[LA_GROUP][DP];
    __shared__ __align__(16) float sa[PER_CHANNEL ? LA_GROUP : 1][PER_CHANNEL ? DP : 4];
    __shared__ float sv[LA_GROUP][COLS];
    __shared__ float part[LA_GROUP][LA_DS][COLS];
    __shared__ int where[3];

    const int tid = threadIdx.x, jl = tid & (LA_COLS - 1), ds = tid / LA_COLS;
    const int h = blockIdx.y, j0 = blockIdx.z * COLS + jl;
    const int D = a.D, Dv = a.Dv, H = a.H;
    int row, first, count;
    if (MODE == 0) {
        row = blockIdx.x; first = a.row_first[row]; count = a.row_lens[row];
    } else {
        if (tid == 0) { la_find_chunk(a.row_first, a.row_lens, a.B, blockIdx.x, row, first, count); where[0] = row; where[1] = first; where[2] = count; }
        __syncthreads();
        row = where[0]; first = where[1]; count = where[2];
    }
    if (count <= 0) return;
    const int d0 = ds * R;

    float S[NC][R];
    float* sp = nullptr;
    if (MODE == 0) sp = a.state + (size_t)a.slots[row] * a.state_stride + (size_t)h * D * Dv;
    if (MODE == 2) sp = a.chunk_state + ((size_t)blockIdx.x * H + h) * D * Dv;
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r)
            S[c][r] = (MODE != 1 && j0 + c * LA_COLS < Dv && d0 + r < D) ? sp[(size_t)(d0 + r) * Dv + j0 + c * LA_COLS] : 0.f;

    const float hd = PER_CHANNEL ? 0.f : a.head_decay[h];
    float A = 1.f;                                       // MODE 1: the product of this chunk's decays on channel tid
    const T* proj = (const T*)a.proj;
    const TZ* zp = (const TZ*)a.z;

    // A group's q, k, a and v are fetched into registers while the group before it is walked, and go to shared memory
    // (activations, scale and the decay's exponentials applied on the way) when that group is done.
    constexpr int NQ = LA_GROUP * DP / LA_THREADS;       // entries of q (and of k, of a) a thread fetches for a group
    float fq[NQ], fk[NQ], fa[PER_CHANNEL ? NQ : 1], fv[NC];
    auto fetch = [&](int g0) {
        const int ng = min(LA_GROUP, count - g0);
#pragma unroll
        for (int n = 0; n < NQ; ++n) {
            const int i = tid + n * LA_THREADS, tb = i / DP, d = i % DP;
            const size_t t = (size_t)(first + g0 + tb);
            const bool on = tb < ng && d < D;
            fq[n] = on ? to_f(proj[t * a.ld + a.q_off + h * D + d]) : 0.f;
            fk[n] = on ? to_f(proj[t * a.ld + a.k_off + h * D + d]) : 0.f;
            if constexpr (PER_CHANNEL) fa[n] = on ? to_f(zp[t * a.z_ld + h * D + d]) : 0.f;
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {                   // LA_GROUP * COLS values of v, LA_THREADS a turn
            const int i = tid + c * LA_THREADS, tb = i / COLS, col = blockIdx.z * COLS + i % COLS;
            fv[c] = (tb < ng && col < Dv) ? to_f(proj[(size_t)(first + g0 + tb) * a.ld + a.v_off + h * Dv + col]) : 0.f;
        }
    };
    fetch(0);
    for (int g0 = 0; g0 < count; g0 += LA_GROUP) {
        const int ng = min(LA_GROUP, count - g0);
        __syncthreads();                                 // the last group's reads of shared memory are done
#pragma unroll
        for (int n = 0; n < NQ; ++n) {
            const int i = tid + n * LA_THREADS, tb = i / DP, d = i % DP;
            const bool on = tb < ng && d < D;
            sq[tb][d] = on ? la_act<FAST>(fq[n], a.act_qk) * a.q_scale : 0.f;
            sk[tb][d] = on ? la_act<FAST>(fk[n], a.act_qk) : 0.f;
            if constexpr (PER_CHANNEL) sa[tb][d] = on ? la_channel_decay(fa[n], a.inv_tau) : 0.f;
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int i = tid + c * LA_THREADS;
            sv[i / COLS][i % COLS] = la_act<FAST>(fv[c], a.act_v);
        }
        __syncthreads();
        if (g0 + LA_GROUP < count) fetch(g0 + LA_GROUP);
        if (MODE == 1 && tid < D) {
            for (int tb = 0; tb < ng; ++tb) { if constexpr (PER_CHANNEL) A *= sa[tb][tid]; else A *= hd; }
        }
        auto token = [&](const int tb) {
            float v[NC], acc[NC][2];
#pragma unroll
            for (int c = 0; c < NC; ++c) { v[c] = sv[tb][c * LA_COLS + jl]; acc[c][0] = 0.f; acc[c][1] = 0.f; }
#pragma unroll
            for (int r = 0; r < R; r += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(&sq[tb][d0 + r]);
                const float4 k4 = *reinterpret_cast<const float4*>(&sk[tb][d0 + r]);
                float4 a4 = make_float4(hd, hd, hd, hd);
                if constexpr (PER_CHANNEL) a4 = *reinterpret_cast<const float4*>(&sa[tb][d0 + r]);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    S[c][r + 0] = fmaf(a4.x, S[c][r + 0], k4.x * v[c]);
                    S[c][r + 1] = fmaf(a4.y, S[c][r + 1], k4.y * v[c]);
                    S[c][r + 2] = fmaf(a4.z, S[c][r + 2], k4.z * v[c]);
                    S[c][r + 3] = fmaf(a4.w, S[c][r + 3], k4.w * v[c]);
                    if (MODE != 1) {                     // two chains a column, so that no sum waits long for the one before it
                        acc[c][0] = fmaf(S[c][r + 0], q4.x, acc[c][0]); acc[c][1] = fmaf(S[c][r + 1], q4.y, acc[c][1]);
                        acc[c][0] = fmaf(S[c][r + 2], q4.z, acc[c][0]); acc[c][1] = fmaf(S[c][r + 3], q4.w, acc[c][1]);
                    }
                }
            }
            if (MODE != 1) {
#pragma unroll
                for (int c = 0; c < NC; ++c) part[tb][ds][c * LA_COLS + jl] = acc[c][0] + acc[c][1];
            }
        };
        if (ng == LA_GROUP) {                            // a full group: constant addresses, no loop
#pragma unroll
            for (int tb = 0; tb < LA_GROUP; ++tb) token(tb);
        } else {
            for (int tb = 0; tb < ng; ++tb) token(tb);
        }
        if (MODE != 1) {
            __syncthreads();
#pragma unroll
            for (int c = 0; c < NC; ++c) {               // LA_GROUP * COLS outputs a group, LA_THREADS a turn
                const int i = tid + c * LA_THREADS, tb = i / COLS, col = blockIdx.z * COLS + i % COLS;
                if (tb < ng && col < Dv) {
                    float o = 0.f;
#pragma unroll
                    for (int s = 0; s < LA_DS; ++s) o += part[tb][s][i % COLS];
                    a.out[(size_t)(first + g0 + tb) * ((size_t)H * Dv) + (size_t)h * Dv + col] = o;
                }
            }
        }
    }
    if (MODE == 0 || MODE == 1) {
        float* dst = MODE == 0 ? sp : a.chunk_state + ((size_t)blockIdx.x * H + h) * D * Dv;
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (j0 + c * LA_COLS < Dv && d0 + r < D) dst[(size_t)(d0 + r) * Dv + j0 + c * LA_COLS] = S[c][r];
        if (MODE == 1 && blockIdx.z == 0 && tid < D) a.chunk_decay[((size_t)blockIdx.x * H + h) * D + tid] = A;
    }
}

// Pass 2: an element of a sequence's state a thread; the sequence's chunks in order.
__global__ void __launch_bounds__(256) la_carry_kernel(LAArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const size_t per = (size_t)a.H * a.D * a.Dv;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    int base = 0;
    for (int i = 0; i < b; ++i) base += (a.row_lens[i] + LA_CHUNK - 1) / LA_CHUNK;
    const int nc = (a.row_lens[b] + LA_CHUNK - 1) / LA_CHUNK;
    if (nc == 0) return;
    const size_t hd = e / a.Dv;                                              // (head, channel)
    float* sp = a.state + (size_t)a.slots[b] * a.state_stride + e;
    float carry = *sp;
    // Eight chunks' contributions and decays are read at once (they do not depend on the carry): one read in flight a thread
    // would leave the memory system idle, a chunk's data being a megabyte away from the next one's.
    for (int c0 = base; c0 < base + nc; c0 += 8) {
        float own[8], dec[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const bool on = c0 + u < base + nc;
            own[u] = on ? a.chunk_state[(size_t)(c0 + u) * per + e] : 0.f;
            dec[u] = on ? a.chunk_decay[(size_t)(c0 + u) * a.H * a.D + hd] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (c0 + u < base + nc) {
                a.chunk_state[(size_t)(c0 + u) * per + e] = carry;
                carry = fmaf(dec[u], carry, own[u]);
            }
        }
    }
    *sp = carry;
}

template <typename T, typename TZ, int R, int NC, bool PC>
static int la_run(const LAArgs& a, int chunked, cudaStream_t s) {
    const int tiles = (a.Dv + LA_COLS * NC - 1) / (LA_COLS * NC);
    if (!chunked) {
        PE_TRY(pe_launch(la_walk_kernel<T, TZ, R, NC, PC, 0>, dim3(a.B, a.H, tiles), LA_THREADS, 0, s, a));
        PE_LAUNCH_CHECK();
        return 0;
    }
    PE_TRY(pe_launch(la_walk_kernel<T, TZ, R, NC, PC, 1>, dim3(a.max_chunks, a.H, tiles), LA_THREADS, 0, s, a));
    PE_LAUNCH_CHECK();
    const size_t per = (size_t)a.H * a.D * a.Dv;
    PE_TRY(pe_launch(la_carry_kernel, dim3((unsigned)((per + 255) / 256), a.B), 256, 0, s, a));
    PE_LAUNCH_CHECK();
    PE_TRY(pe_launch(la_walk_kernel<T, TZ, R, NC, PC, 2>, dim3(a.max_chunks, a.H, tiles), LA_THREADS, 0, s, a));
    PE_LAUNCH_CHECK();
    return 0;
}

// Two columns a thread where the state is at least 64 columns wide and a thread's rows leave the registers for it.
template <typename T, typename TZ, bool PC>
static int la_by_rows(const LAArgs& a, int chunked, cudaStream_t s) {
    const bool two = a.Dv >= 64;
    if (a.D <= 8 * LA_DS) return two ? la_run<T, TZ, 8, 2, PC>(a, chunked, s) : la_run<T, TZ, 8, 1, PC>(a, chunked, s);
    if (a.D <= 16 * LA_DS) return two ? la_run<T, TZ, 16, 2, PC>(a, chunked, s) : la_run<T, TZ, 16, 1, PC>(a, chunked, s);
    if (a.D <= 32 * LA_DS) return la_run<T, TZ, 32, 1, PC>(a, chunked, s);
    return PE_ERR_UNSUPPORTED;
}

// Chunks a step of T tokens in B sequences can have at most.
extern "C" int pe_linear_attention_chunks(int T, int B) { return (T + LA_CHUNK - 1) / LA_CHUNK + B; }

// Floats of scratch the chunked way needs.
extern "C" long long pe_linear_attention_scratch_floats(int T, int B, int H, int D, int Dv) {
    return (long long)pe_linear_attention_chunks(T, B) * H * D * ((long long)Dv + 1);
}

extern "C" int pe_linear_attention(const void* proj, int dtype, int ld, int q_off, int k_off, int v_off, const void* z, int z_dtype,
                                   int z_ld, const float* head_decay, float inv_tau, float q_scale, int act_qk, int act_v,
                                   float* state, long long state_stride, const int* row_first, const int* row_lens,
                                   const int* slots, float* out, int T, int B, int H, int D, int Dv, int chunked, float* scratch,
                                   void* stream) {
    if (T <= 0 || B <= 0) return 0;
    if ((z == nullptr) == (head_decay == nullptr) || D <= 0 || Dv <= 0 || H <= 0) return PE_ERR_UNSUPPORTED;
    if (chunked && !scratch) return PE_ERR_UNSUPPORTED;
    LAArgs a;
    a.proj = proj; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
    a.z = z; a.z_ld = z_ld; a.head_decay = head_decay; a.inv_tau = inv_tau; a.q_scale = q_scale;
    a.act_qk = act_qk; a.act_v = act_v; a.state = state; a.state_stride = state_stride;
    a.row_first = row_first; a.row_lens = row_lens; a.slots = slots; a.out = out;
    a.B = B; a.H = H; a.D = D; a.Dv = Dv;
    a.max_chunks = pe_linear_attention_chunks(T, B);
    a.chunk_state = scratch;
    a.chunk_decay = scratch ? scratch + (size_t)a.max_chunks * H * D * Dv : nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    const bool pc = z != nullptr;
    if (dtype == PE_F32) {
        if (!pc) return la_by_rows<float, float, false>(a, chunked, s);
        if (z_dtype == PE_F32) return la_by_rows<float, float, true>(a, chunked, s);
        return PE_ERR_UNSUPPORTED;
    }
    if (dtype == PE_BF16) {
        if (!pc) return la_by_rows<bf16, bf16, false>(a, chunked, s);
        if (z_dtype == PE_F32) return la_by_rows<bf16, float, true>(a, chunked, s);
    }
    return PE_ERR_UNSUPPORTED;
}
