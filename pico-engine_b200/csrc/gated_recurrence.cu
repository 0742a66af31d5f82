// The minGRU recurrence on the projections of a step's tokens.
//
//   z = sigmoid(pz)      c = pu + 1/2 where pu >= 0, sigmoid(pu) elsewhere      S_t = (1 - z) S_(t-1) + z c
//   y_t = S_t * silu(pg)
//
// `proj` [T, 3W] holds pz | pu | pg of every token (biases added by the product that made them); gates,
// candidate, state and y are float32, y is stored in the step's dtype.  S of a sequence lives in its slot of
// the float32 state area (`state` points at channel 0 of slot 0, slots `state_stride` floats apart) and is
// zero for a new sequence.
//
// Two ways to run it, with the same result up to float32 rounding:
//  * sequential: thread per (sequence, channel), its tokens one after the other: a step of single tokens.
//  * chunked: the recurrence is linear, S_end = A * S_in + B with A = prod (1 - z), so the packed tokens are cut
//    into chunks of MG_CHUNK; pass 1 gives every chunk its (A, B) from S_in = 0, pass 2 walks a channel's chunks
//    in order and hands each its S_in, pass 3 runs each chunk again from its S_in and writes y.  A sequence's
//    first token of the step restarts the chain from the sequence's stored state (a chunk may hold the end of
//    one sequence and the start of the next), which makes it a segmented scan over the packed tokens.  Pass 1
//    copies the stored state it meets into `snap` [B, W], because pass 3 stores new states while other blocks
//    of pass 3 would still read the old ones.
#include "common.cuh"

#define MG_CHUNK 16
#define MG_THREADS 128

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T>
__device__ __forceinline__ void mg_gates(const T* proj_row, int W, int ch, float& a, float& zc, float& gate) {
    const float pz = to_f(proj_row[ch]), pu = to_f(proj_row[W + ch]), pg = to_f(proj_row[2 * (size_t)W + ch]);
    const float z = sigmoid_f(pz);
    const float c = pu >= 0.f ? pu + 0.5f : sigmoid_f(pu);
    a = 1.0f - z;
    zc = z * c;
    gate = pg * sigmoid_f(pg);
}

template <typename T>
__global__ void __launch_bounds__(MG_THREADS) mingru_sequential_kernel(const T* proj, float* state, long long state_stride,
                                                                       const int* row_first, const int* row_lens, const int* slots,
                                                                       T* y, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, ch = blockIdx.y * MG_THREADS + threadIdx.x;
    if (ch >= W) return;
    const int first = row_first[b], n = row_lens[b];
    float* sp = state + (size_t)slots[b] * state_stride + ch;
    float S = *sp;
    for (int t = first; t < first + n; ++t) {
        float a, zc, gate;
        mg_gates(proj + (size_t)t * 3 * W, W, ch, a, zc, gate);
        S = fmaf(a, S, zc);
        y[(size_t)t * W + ch] = from_f<T>(S * gate);
    }
    *sp = S;
}

#define MG_BATCH 16     // tokens whose projections a thread loads before it walks them: the loads are in flight together

template <typename T>
__device__ __forceinline__ void mg_load(const T* proj, int t, int n, int W, int ch, float (&pz)[MG_BATCH], float (&pu)[MG_BATCH], float (&pg)[MG_BATCH]) {
#pragma unroll
    for (int k = 0; k < MG_BATCH; ++k) {
        if (k < n) {
            const T* row = proj + (size_t)(t + k) * 3 * W;
            pz[k] = to_f(row[ch]); pu[k] = to_f(row[W + ch]); pg[k] = to_f(row[2 * (size_t)W + ch]);
        }
    }
}
__device__ __forceinline__ void mg_gate_values(float pz, float pu, float& a, float& zc) {
    const float z = sigmoid_f(pz);
    a = 1.0f - z;
    zc = z * (pu >= 0.f ? pu + 0.5f : sigmoid_f(pu));
}

// pass 1: (A, B) of every chunk; `carry` [chunks, 2, W]
template <typename T>
__global__ void __launch_bounds__(MG_THREADS) mingru_chunk_kernel(const T* proj, const float* state, long long state_stride,
                                                                  const int* tok_row, const int* row_first, const int* slots,
                                                                  float* carry, float* snap, int Ttot, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int k = blockIdx.x, ch = blockIdx.y * MG_THREADS + threadIdx.x;
    if (ch >= W) return;
    const int t0 = k * MG_CHUNK, t1 = min(Ttot, t0 + MG_CHUNK);
    float A = 1.f, Bv = 0.f;
    for (int tb = t0; tb < t1; tb += MG_BATCH) {
        float pz[MG_BATCH], pu[MG_BATCH], pg[MG_BATCH];
        const int n = min(MG_BATCH, t1 - tb);
        mg_load(proj, tb, n, W, ch, pz, pu, pg);
#pragma unroll
        for (int j = 0; j < MG_BATCH; ++j) {
            if (j < n) {
                const int t = tb + j;
                float a, zc;
                mg_gate_values(pz[j], pu[j], a, zc);
                const int b = tok_row[t];
                if (t == row_first[b]) {                     // restart from the sequence's stored state
                    const float s_in = state[(size_t)slots[b] * state_stride + ch];
                    snap[(size_t)b * W + ch] = s_in;
                    A = 0.f;
                    Bv = fmaf(a, s_in, zc);
                } else {
                    A *= a;
                    Bv = fmaf(a, Bv, zc);
                }
            }
        }
    }
    carry[((size_t)k * 2) * W + ch] = A;
    carry[((size_t)k * 2 + 1) * W + ch] = Bv;
}

// pass 2: carry[k][0] <- S_in of chunk k (the pairs of 8 chunks are loaded before they are walked)
__global__ void __launch_bounds__(MG_THREADS) mingru_carry_kernel(float* carry, int chunks, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int ch = blockIdx.x * MG_THREADS + threadIdx.x;
    if (ch >= W) return;
    float S = 0.f;
    for (int kb = 0; kb < chunks; kb += MG_BATCH) {
        float A[MG_BATCH], Bv[MG_BATCH];
        const int n = min(MG_BATCH, chunks - kb);
#pragma unroll
        for (int j = 0; j < MG_BATCH; ++j)
            if (j < n) { A[j] = carry[((size_t)(kb + j) * 2) * W + ch]; Bv[j] = carry[((size_t)(kb + j) * 2 + 1) * W + ch]; }
#pragma unroll
        for (int j = 0; j < MG_BATCH; ++j)
            if (j < n) { carry[((size_t)(kb + j) * 2) * W + ch] = S; S = fmaf(A[j], S, Bv[j]); }
    }
}

// pass 3: every chunk again from its S_in; y and the new states
template <typename T>
__global__ void __launch_bounds__(MG_THREADS) mingru_apply_kernel(const T* proj, float* state, long long state_stride,
                                                                  const int* tok_row, const int* row_first, const int* slots,
                                                                  const float* carry, const float* snap, T* y, int Ttot, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int k = blockIdx.x, ch = blockIdx.y * MG_THREADS + threadIdx.x;
    if (ch >= W) return;
    const int t0 = k * MG_CHUNK, t1 = min(Ttot, t0 + MG_CHUNK);
    float S = carry[((size_t)k * 2) * W + ch];
    for (int tb = t0; tb < t1; tb += MG_BATCH) {
        float pz[MG_BATCH], pu[MG_BATCH], pg[MG_BATCH];
        const int n = min(MG_BATCH, t1 - tb);
        mg_load(proj, tb, n, W, ch, pz, pu, pg);
#pragma unroll
        for (int j = 0; j < MG_BATCH; ++j) {
            if (j < n) {
                const int t = tb + j;
                float a, zc;
                mg_gate_values(pz[j], pu[j], a, zc);
                const int b = tok_row[t];
                if (t == row_first[b]) S = snap[(size_t)b * W + ch];
                S = fmaf(a, S, zc);
                y[(size_t)t * W + ch] = from_f<T>(S * (pg[j] * sigmoid_f(pg[j])));
                if (t + 1 == row_first[b + 1]) state[(size_t)slots[b] * state_stride + ch] = S;      // the sequence's last token of the step
            }
        }
    }
}

extern "C" long long pe_mingru_scratch_floats(int T, int B, int W) {
    const long long chunks = (T + MG_CHUNK - 1) / MG_CHUNK;
    return (chunks * 2 + B) * (long long)W;
}

extern "C" int pe_mingru(const void* proj, int dtype, float* state, long long state_stride, const int* tok_row,
                         const int* row_first, const int* row_lens, const int* slots, void* y, int T, int B, int W,
                         int chunked, float* scratch, void* stream) {
    if (T <= 0 || B <= 0) return 0;
    if (dtype != PE_F32 && dtype != PE_BF16) return PE_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned cb = (W + MG_THREADS - 1) / MG_THREADS;
    if (!chunked) {
        if (dtype == PE_F32) PE_TRY(pe_launch(mingru_sequential_kernel<float>, dim3(B, cb), MG_THREADS, 0, s, (const float*)proj, state, state_stride, row_first, row_lens, slots, (float*)y, W));
        else PE_TRY(pe_launch(mingru_sequential_kernel<bf16>, dim3(B, cb), MG_THREADS, 0, s, (const bf16*)proj, state, state_stride, row_first, row_lens, slots, (bf16*)y, W));
        PE_LAUNCH_CHECK();
        return 0;
    }
    if (scratch == nullptr) return PE_ERR_UNSUPPORTED;
    const int chunks = (T + MG_CHUNK - 1) / MG_CHUNK;
    float* carry = scratch;
    float* snap = scratch + (size_t)chunks * 2 * W;
    if (dtype == PE_F32) PE_TRY(pe_launch(mingru_chunk_kernel<float>, dim3(chunks, cb), MG_THREADS, 0, s, (const float*)proj, (const float*)state, state_stride, tok_row, row_first, slots, carry, snap, T, W));
    else PE_TRY(pe_launch(mingru_chunk_kernel<bf16>, dim3(chunks, cb), MG_THREADS, 0, s, (const bf16*)proj, (const float*)state, state_stride, tok_row, row_first, slots, carry, snap, T, W));
    PE_LAUNCH_CHECK();
    PE_TRY(pe_launch(mingru_carry_kernel, cb, MG_THREADS, 0, s, carry, chunks, W));
    PE_LAUNCH_CHECK();
    if (dtype == PE_F32) PE_TRY(pe_launch(mingru_apply_kernel<float>, dim3(chunks, cb), MG_THREADS, 0, s, (const float*)proj, state, state_stride, tok_row, row_first, slots, (const float*)carry, (const float*)snap, (float*)y, T, W));
    else PE_TRY(pe_launch(mingru_apply_kernel<bf16>, dim3(chunks, cb), MG_THREADS, 0, s, (const bf16*)proj, state, state_stride, tok_row, row_first, slots, (const float*)carry, (const float*)snap, (bf16*)y, T, W));
    PE_LAUNCH_CHECK();
    return 0;
}
