// A gated linear recurrence over channels (the recurrent unit of Griffin-style blocks), for steps that mix
// portions of prompts and single tokens.  For every request the step brings tokens cu_q[s] .. cu_q[s+1]-1; what
// the request keeps between steps lies in state slots (float): the last K-1 inputs of the short convolution and
// the recurrence's state, both zero when the request begins.
//
//   acv_causal_conv     u[t][c] = cb[c] + sum_j w[c][K-1-j] * (x[t-j][c] + xb[c])          j = 0 .. K-1, float
//   acv_block_gates     r = sigmoid(A_b u_b + a_b),  g = sigmoid(B_b u_b + b_b)            per block b of the channels, float
//                       a = exp(c_r * r * sp[c]),    b = sqrt(1 - a^2) * g * u             what the recurrence multiplies and adds
//   acv_gated_scan      S = a S + b;  out = S * gelu_tanh(y + yb)
//
// sp[c] is softplus of the channel's decay parameter (folded when the weights are loaded), c_r the design's
// constant (negative).  1 - a^2 is taken as -expm1(2 log a), which keeps its digits where a is close to 1.
// Everything here is 32-bit; only the inputs x and y (a projection's output) and the result may have the run's
// element type.
//
// The recurrence is linear in S, so a long portion is cut into segments of seg_len tokens that run side by side
// (the step's list of (request, segment) items): a first launch leaves each segment's (product of a, state reached
// from zero; the first segment starts from the request's state), a small one folds them into what lies in front of
// every segment, and a last one walks the segments again from there, writing the outputs.  Steps of short portions and single tokens run the second launch alone.
#include "mma_tiles.cuh"

// ----------------------------------------------------------------------------- short causal convolution per channel
// grid (tokens, channel tiles).  The tokens that reach back into the state (the first K-1 of a request's portion)
// are all computed by the block of the portion's first token, which then replaces the state: each channel's
// state is read and written by one thread only.
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ xb,
                                   const float* __restrict__ w, const float* __restrict__ cb, float* __restrict__ state,
                                   const int* __restrict__ slots, const int* __restrict__ cu_q,
                                   const int* __restrict__ seq_of_token, float* __restrict__ u, int C, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seq = seq_of_token[t];
    const int first = cu_q[seq], len = cu_q[seq + 1] - first;
    const int off = t - first;
    const float bias_in = xb ? xb[c] : 0.f;
    const float* wc = w + (size_t)c * K;
    if (off >= K - 1) {
        float acc = cb ? cb[c] : 0.f;
        for (int j = 0; j < K; ++j) acc = fmaf(wc[K - 1 - j], to_f32(x[(size_t)(t - j) * ldx + c]) + bias_in, acc);
        u[(size_t)t * C + c] = acc;
        return;
    }
    if (off != 0) return;
    float* st = state + (size_t)slots[seq] * (K - 1) * C;      // [K-1][C], the oldest input first
    const int n_here = len < K - 1 ? len : K - 1;
    for (int n = 0; n < n_here; ++n) {
        float acc = cb ? cb[c] : 0.f;
        for (int j = 0; j < K; ++j) {
            const int src = n - j;
            const float v = src >= 0 ? to_f32(x[(size_t)(first + src) * ldx + c]) + bias_in : st[(size_t)(K - 1 + src) * C + c];
            acc = fmaf(wc[K - 1 - j], v, acc);
        }
        u[(size_t)(first + n) * C + c] = acc;
    }
    for (int i = 0; i < K - 1; ++i) {       // ascending: what is read lies behind what has been written
        const int src = len - (K - 1) + i;
        st[(size_t)i * C + c] = src >= 0 ? to_f32(x[(size_t)(first + src) * ldx + c]) + bias_in : st[(size_t)(len + i) * C + c];
    }
}

// The same for float inputs with four neighbouring channels to a thread (16-byte loads and stores): C and the row
// stride multiples of four, x, the state and u aligned to 16 bytes.  wt: the taps transposed, [K][C], so that the four
// channels' taps of one lag are one vector as well.
__device__ __forceinline__ float4 f4_add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 f4_fma(float4 w, float4 v, float4 acc) {
    return make_float4(fmaf(w.x, v.x, acc.x), fmaf(w.y, v.y, acc.y), fmaf(w.z, v.z, acc.z), fmaf(w.w, v.w, acc.w));
}

__global__ void causal_conv4_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ xb,
                                    const float* __restrict__ wt, const float* __restrict__ cb, float* __restrict__ state,
                                    const int* __restrict__ slots, const int* __restrict__ cu_q,
                                    const int* __restrict__ seq_of_token, float* __restrict__ u, int C, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= C) return;
    const int seq = seq_of_token[t];
    const int first = cu_q[seq], len = cu_q[seq + 1] - first;
    const int off = t - first;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 bias_in = xb ? *reinterpret_cast<const float4*>(xb + c) : zero;
    const float4 bias_out = cb ? *reinterpret_cast<const float4*>(cb + c) : zero;
    auto tap = [&](int j) { return *reinterpret_cast<const float4*>(wt + (size_t)j * C + c); };     // the j-th tap of the four channels
    auto in = [&](int row) { return f4_add(*reinterpret_cast<const float4*>(x + (size_t)row * ldx + c), bias_in); };
    if (off >= K - 1) {
        float4 acc = bias_out;
        for (int j = 0; j < K; ++j) acc = f4_fma(tap(K - 1 - j), in(t - j), acc);
        *reinterpret_cast<float4*>(u + (size_t)t * C + c) = acc;
        return;
    }
    if (off != 0) return;
    float* st = state + (size_t)slots[seq] * (K - 1) * C;      // [K-1][C], the oldest input first
    const int n_here = len < K - 1 ? len : K - 1;
    for (int n = 0; n < n_here; ++n) {
        float4 acc = bias_out;
        for (int j = 0; j < K; ++j) {
            const int src = n - j;
            const float4 v = src >= 0 ? in(first + src) : *reinterpret_cast<const float4*>(st + (size_t)(K - 1 + src) * C + c);
            acc = f4_fma(tap(K - 1 - j), v, acc);
        }
        *reinterpret_cast<float4*>(u + (size_t)(first + n) * C + c) = acc;
    }
    for (int i = 0; i < K - 1; ++i) {       // ascending: what is read lies behind what has been written
        const int src = len - (K - 1) + i;
        const float4 v = src >= 0 ? in(first + src) : *reinterpret_cast<const float4*>(st + (size_t)(len + i) * C + c);
        *reinterpret_cast<float4*>(st + (size_t)i * C + c) = v;
    }
}

// w: the taps [C][K]; wt (may be null): the same transposed, [K][C], which the form with four channels to a thread reads
ACV_API int acv_causal_conv(const void* x, int ldx, const float* xb, const float* w, const float* cb, float* state,
                            const int* slots, const int* cu_q, const int* seq_of_token, float* u, int T, int C, int K,
                            int dtype, const float* wt, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (C <= 0 || K < 1) return ACV_ERR_SIZE;
    dim3 grid(T, (C + 127) / 128);
    const bool four = wt && !((uintptr_t)wt & 15) && dtype == ACV_F32 && C % 4 == 0 && ldx % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)u & 15) &&
                      !((uintptr_t)state & 15) && (!xb || !((uintptr_t)xb & 15)) && (!cb || !((uintptr_t)cb & 15));
    if (four)
        acv_launch(PDL_MISC, causal_conv4_kernel, dim3(T, (C / 4 + 127) / 128), 128, 0, stream, (const float*)x, ldx, xb, wt, cb,
                   state, slots, cu_q, seq_of_token, u, C, K);
    else if (dtype == ACV_F32)
        acv_launch(PDL_MISC, causal_conv_kernel<float>, grid, 128, 0, stream, (const float*)x, ldx, xb, w, cb, state, slots,
                   cu_q, seq_of_token, u, C, K);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_MISC, causal_conv_kernel<bf16>, grid, 128, 0, stream, (const bf16*)x, ldx, xb, w, cb, state, slots,
                   cu_q, seq_of_token, u, C, K);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- the two gates, block-diagonal
// wa, wb: [blocks][in][out] (transposed when loaded, so that the threads of a warp read neighbouring outputs).
// grid (token tiles of GT, blocks, tiles of 64 outputs); a thread owns one output of its block for all tokens of the
// tile.  The tile's inputs wait in shared memory as [in][token], so that a thread reads the GT tokens of an input as
// vectors of four (one shared-memory instruction to eight multiply-adds).
template <int GT>
__global__ void block_gates_kernel(const float* __restrict__ u, const float* __restrict__ wa, const float* __restrict__ ba,
                                   const float* __restrict__ wb, const float* __restrict__ bb,
                                   const float* __restrict__ sp, float c_r, float* __restrict__ r,
                                   float* __restrict__ g, int T, int C, int BW) {
    extern __shared__ __align__(16) float su[];          // [BW][GT]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * GT, blk = blockIdx.y;
    const int nt = min(GT, T - t0);
    for (int i = threadIdx.x; i < GT * BW; i += blockDim.x) {
        const int tt = i / BW, e = i - tt * BW;
        su[e * GT + tt] = tt < nt ? u[(size_t)(t0 + tt) * C + blk * BW + e] : 0.f;
    }
    __syncthreads();
    const int o = blockIdx.z * blockDim.x + threadIdx.x;
    if (o >= BW) return;
    const float* wa_b = wa + (size_t)blk * BW * BW + o;
    const float* wb_b = wb + (size_t)blk * BW * BW + o;
    float ar[GT], ag[GT];
#pragma unroll
    for (int tt = 0; tt < GT; ++tt) ar[tt] = ag[tt] = 0.f;
#pragma unroll 4
    for (int i = 0; i < BW; ++i) {
        const float a = wa_b[(size_t)i * BW], b = wb_b[(size_t)i * BW];
        const float4* x4 = reinterpret_cast<const float4*>(su + i * GT);
#pragma unroll
        for (int q = 0; q < GT / 4; ++q) {
            const float4 x = x4[q];
            ar[4 * q] = fmaf(a, x.x, ar[4 * q]); ar[4 * q + 1] = fmaf(a, x.y, ar[4 * q + 1]);
            ar[4 * q + 2] = fmaf(a, x.z, ar[4 * q + 2]); ar[4 * q + 3] = fmaf(a, x.w, ar[4 * q + 3]);
            ag[4 * q] = fmaf(b, x.x, ag[4 * q]); ag[4 * q + 1] = fmaf(b, x.y, ag[4 * q + 1]);
            ag[4 * q + 2] = fmaf(b, x.z, ag[4 * q + 2]); ag[4 * q + 3] = fmaf(b, x.w, ag[4 * q + 3]);
        }
    }
    const int ch = blk * BW + o;
    const float b1 = ba ? ba[ch] : 0.f, b2 = bb ? bb[ch] : 0.f;
    const float rate = c_r * sp[ch];
#pragma unroll
    for (int tt = 0; tt < GT; ++tt) {
        if (tt < nt) {
            const float rr = 1.f / (1.f + expf(-(ar[tt] + b1)));
            const float gg = 1.f / (1.f + expf(-(ag[tt] + b2)));
            const float la = rate * rr;                    // log a <= 0
            r[(size_t)(t0 + tt) * C + ch] = expf(la);
            g[(size_t)(t0 + tt) * C + ch] = sqrtf(fmaxf(-expm1f(2.f * la), 0.f)) * gg * su[o * GT + tt];
        }
    }
}

// r <- a, g <- b of the recurrence (see the head of the file)
ACV_API int acv_block_gates(const float* u, const float* wa, const float* ba, const float* wb, const float* bb,
                            const float* sp, float c_r, float* r, float* g, int T, int C, int blocks, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (blocks <= 0 || C % blocks) return ACV_ERR_SIZE;
    const int BW = C / blocks;
    const int gt = T <= 512 ? 4 : 16;       // few tokens: small tiles, so that the grid still fills the device
    const size_t smem = (size_t)gt * BW * sizeof(float);
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    static AcvSmemConfig cfg4, cfg16;
    if (smem > 48 * 1024) {
        const int e = gt == 4 ? acv_ensure_smem(cfg4, block_gates_kernel<4>, (int)smem)
                              : acv_ensure_smem(cfg16, block_gates_kernel<16>, (int)smem);
        if (e) return e;
    }
    const int threads = BW >= 64 ? 64 : 32;
    dim3 grid((T + gt - 1) / gt, blocks, (BW + threads - 1) / threads);
    if (gt == 4)
        acv_launch(PDL_MISC, block_gates_kernel<4>, grid, threads, smem, stream, u, wa, ba, wb, bb, sp, c_r, r, g, T, C, BW);
    else
        acv_launch(PDL_MISC, block_gates_kernel<16>, grid, threads, smem, stream, u, wa, ba, wb, bb, sp, c_r, r, g, T, C, BW);
    return acv_launch_status();
}

// The same on the tensor cores, for runs whose projections are bfloat16: the inputs u are rounded to bfloat16 for the
// two products (float accumulation); sigmoid, decay and b stay float and b takes the unrounded u.  wa, wb: bfloat16
// [blocks][out][in] as the weight file has them.  grid (tiles of 64 tokens, blocks, tiles of OT outputs), four warps
// of 16 tokens; the tile of u and the weights' 2 x OT rows wait in shared memory with rows padded by 16 bytes.  OT is 64,
// or 16 for steps of few tokens, whose grid would otherwise be a few blocks that each wait for 2 x 64 rows of weights.
template <int OT>
__global__ void __launch_bounds__(128) block_gates_mma_kernel(const float* __restrict__ u, const bf16* __restrict__ wa,
                                                             const float* __restrict__ ba, const bf16* __restrict__ wb,
                                                             const float* __restrict__ bb, const float* __restrict__ sp,
                                                             float c_r, float* __restrict__ r, float* __restrict__ g,
                                                             int T, int C, int BW) {
    extern __shared__ __align__(16) unsigned char gm_smem[];
    const int LD = BW + 8;                                      // elements of a padded row
    bf16* As = reinterpret_cast<bf16*>(gm_smem);                // [64][LD]
    bf16* Bs = As + 64 * LD;                                    // [2][OT][LD]
    float* cs = reinterpret_cast<float*>(Bs + 2 * OT * LD);     // [3][OT]: the two biases and the rate of the tile's outputs
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * 64, blk = blockIdx.y, o0 = blockIdx.z * OT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quads = BW / 4;                                   // 16-byte pieces of a row of u
#pragma unroll 4
    for (int i = tid; i < 64 * quads; i += 128) {
        const int tt = i / quads, e = (i - tt * quads) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t0 + tt < T) v = *reinterpret_cast<const float4*>(u + (size_t)(t0 + tt) * C + blk * BW + e);
        *reinterpret_cast<uint2*>(As + tt * LD + e) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
    }
    if (tid < OT) {
        const int ch = blk * BW + o0 + tid;
        const bool in = o0 + tid < BW;
        cs[tid] = in && ba ? ba[ch] : 0.f;
        cs[OT + tid] = in && bb ? bb[ch] : 0.f;
        cs[2 * OT + tid] = in ? c_r * sp[ch] : 0.f;
    }
    const int chunks = BW / 8;                                  // 16-byte pieces of a weight row
    for (int i = tid; i < 2 * OT * chunks; i += 128) {
        const int q = i / (OT * chunks), rem = i - q * OT * chunks;
        const int row = rem / chunks, ch = rem - row * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (o0 + row < BW)
            v = *reinterpret_cast<const uint4*>((q ? wb : wa) + ((size_t)blk * BW + o0 + row) * BW + ch * 8);
        *reinterpret_cast<uint4*>(Bs + ((size_t)q * OT + row) * LD + ch * 8) = v;
    }
    __syncthreads();
    const int gr = lane >> 2, tq = lane & 3;
    constexpr int NT = OT / 8;                                  // output tiles of eight
    float acc[2][NT][4];
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[q][j][e] = 0.f;
    const bf16* a_row = As + (warp * 16 + gr) * LD + 2 * tq;
    for (int k0 = 0; k0 < BW; k0 += 16) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(a_row + k0);
        a[1] = *reinterpret_cast<const uint32_t*>(a_row + 8 * LD + k0);
        a[2] = *reinterpret_cast<const uint32_t*>(a_row + k0 + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(a_row + 8 * LD + k0 + 8);
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const bf16* b_row = Bs + ((size_t)q * OT + j * 8 + gr) * LD + k0 + 2 * tq;
                mma_bf16(acc[q][j], a, *reinterpret_cast<const uint32_t*>(b_row), *reinterpret_cast<const uint32_t*>(b_row + 8));
            }
    }
    // the unrounded inputs of this thread's outputs: all loads first, so that they do not wait for one another
    float2 uu[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int t = t0 + warp * 16 + gr + hh * 8, o = o0 + j * 8 + 2 * tq;
            uu[j][hh] = t < T && o < BW ? *reinterpret_cast<const float2*>(u + (size_t)t * C + blk * BW + o) : make_float2(0.f, 0.f);
        }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int t = t0 + warp * 16 + gr + hh * 8;
            const int ol = j * 8 + 2 * tq;                      // the first of this thread's two neighbouring outputs
            if (t < T && o0 + ol < BW) {
                float av[2], bv[2];
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int e = hh * 2 + x;
                    const float rr = 1.f / (1.f + expf(-(acc[0][j][e] + cs[ol + x])));
                    const float gg = 1.f / (1.f + expf(-(acc[1][j][e] + cs[OT + ol + x])));
                    const float la = cs[2 * OT + ol + x] * rr;
                    av[x] = expf(la);
                    bv[x] = sqrtf(fmaxf(-expm1f(2.f * la), 0.f)) * gg * (x ? uu[j][hh].y : uu[j][hh].x);
                }
                const size_t at = (size_t)t * C + blk * BW + o0 + ol;
                *reinterpret_cast<float2*>(r + at) = make_float2(av[0], av[1]);
                *reinterpret_cast<float2*>(g + at) = make_float2(bv[0], bv[1]);
            }
        }
}

// takes blocks whose width is a multiple of 16 up to 256 and 16-byte aligned weights
ACV_API int acv_block_gates_mma(const float* u, const void* wa, const float* ba, const void* wb, const float* bb,
                                const float* sp, float c_r, float* r, float* g, int T, int C, int blocks, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (blocks <= 0 || C % blocks) return ACV_ERR_SIZE;
    const int BW = C / blocks;
    if (BW % 16 || BW > 256) return ACV_ERR_SIZE;
    if (((uintptr_t)wa & 15) || ((uintptr_t)wb & 15) || ((uintptr_t)u & 15) || ((uintptr_t)r & 7) || ((uintptr_t)g & 7)) return ACV_ERR_ALIGN;
    const int ot = T <= 128 ? 16 : 64;
    const int smem = (64 + 2 * ot) * (BW + 8) * 2 + 3 * ot * 4;
    static AcvSmemConfig cfg64, cfg16;
    if (smem > 48 * 1024) {
        const int e = ot == 64 ? acv_ensure_smem(cfg64, block_gates_mma_kernel<64>, smem)
                               : acv_ensure_smem(cfg16, block_gates_mma_kernel<16>, smem);
        if (e) return e;
    }
    dim3 grid((T + 63) / 64, blocks, (BW + ot - 1) / ot);
    if (ot == 64)
        acv_launch(PDL_MISC, block_gates_mma_kernel<64>, grid, 128, smem, stream, u, (const bf16*)wa, ba, (const bf16*)wb, bb,
                   sp, c_r, r, g, T, C, BW);
    else
        acv_launch(PDL_MISC, block_gates_mma_kernel<16>, grid, 128, smem, stream, u, (const bf16*)wa, ba, (const bf16*)wb, bb,
                   sp, c_r, r, g, T, C, BW);
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- the recurrence
__device__ __forceinline__ float gelu_tanh_f32(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// grid (items, channel tiles): a thread walks its channel through the item's tokens; the loads of SC tokens are issued
// before their recurrence runs, so that they do not wait for one another.  An item is a segment of a request's portion:
// tokens cu_q[seq] + z * seg_len .. (seg_len of them, or what is left).
#define SC 8

// Between the two launches: the entries (A, B) of a request's segments become, in their B, the states in front of the
// segments that follow: S_in(z + 1) = A(z) S_in(z) + B(z), in place.  grid (items, channel tiles); the block of a
// request's first segment walks the request's entries.
__global__ void scan_fold_kernel(float* __restrict__ seg, const int* __restrict__ seg_seq, const int* __restrict__ seg_idx,
                                 int seg_len, const int* __restrict__ cu_q, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C || seg_idx[item] != 0) return;
    const int seq = seg_seq[item];
    const int nseg = (cu_q[seq + 1] - cu_q[seq] + seg_len - 1) / seg_len;
    float S = seg[((size_t)item * 2 + 1) * C + c];              // the first segment began at the request's state
    for (int z0 = 1; z0 < nseg - 1; z0 += 8) {                  // eight entries' loads at a time
        float A[8], B[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float* e = seg + (size_t)(item + z0 + k) * 2 * C;
            const bool in = z0 + k < nseg - 1;
            A[k] = in ? e[c] : 0.f;
            B[k] = in ? e[C + c] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (z0 + k < nseg - 1) {
                S = fmaf(A[k], S, B[k]);
                seg[((size_t)(item + z0 + k) * 2 + 1) * C + c] = S;
            }
        }
    }
}

// SUMMARY: leave (A, B) of the segment in seg[item] and write no output (the last segment of a request does nothing)
template <typename TY, typename T, bool SUMMARY>
__global__ void gated_scan_kernel(const float* __restrict__ a, const float* __restrict__ b, const TY* __restrict__ y, int ldy,
                                  const float* __restrict__ yb, float* __restrict__ state, const int* __restrict__ slots,
                                  const int* __restrict__ cu_q, const int* __restrict__ seg_seq,
                                  const int* __restrict__ seg_idx, int seg_len, float* __restrict__ seg,
                                  T* __restrict__ out, int ldo, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seq = seg_seq ? seg_seq[item] : item, z = seg_idx ? seg_idx[item] : 0;
    const int q0 = cu_q[seq], q1 = cu_q[seq + 1];
    const int t0 = q0 + z * seg_len, t1 = min(q1, t0 + seg_len);
    if (t1 <= t0) return;
    const bool last = t1 == q1;
    if (SUMMARY && last) return;
    float* st = state + (size_t)slots[seq] * C + c;
    // The request's state as this step found it: read from its slot by the first launch (and by a request's only
    // segment), which also leaves it in the unused entry of the request's last segment for the second launch, whose
    // last segment replaces the slot while its first one may not have begun.
    const int last_item = item - z + (q1 - q0 + seg_len - 1) / seg_len - 1;
    float S;
    if (z == 0) {
        S = (SUMMARY || last) ? *st : seg[((size_t)last_item * 2) * C + c];
        if (SUMMARY) seg[((size_t)last_item * 2) * C + c] = S;
    } else {
        S = SUMMARY ? 0.f : seg[((size_t)(item - 1) * 2 + 1) * C + c];     // what lies in front, after the fold
    }
    float A = 1.f;
    const float bias_y = yb ? yb[c] : 0.f;
    for (int t = t0; t < t1; t += SC) {
        float aa[SC], bb[SC], yy[SC];
#pragma unroll
        for (int i = 0; i < SC; ++i) {
            const bool in = t + i < t1;
            const size_t at = (size_t)(in ? t + i : t) * C + c;
            aa[i] = a[at];
            bb[i] = b[at];
            if (!SUMMARY) yy[i] = gelu_tanh_f32(to_f32(y[(size_t)(in ? t + i : t) * ldy + c]) + bias_y);
        }
#pragma unroll
        for (int i = 0; i < SC; ++i) {
            if (t + i < t1) {
                S = fmaf(aa[i], S, bb[i]);
                if (SUMMARY) A *= aa[i];
                else out[(size_t)(t + i) * ldo + c] = from_f32<T>(S * yy[i]);
            }
        }
    }
    if (SUMMARY) {
        seg[((size_t)item * 2) * C + c] = A;
        seg[((size_t)item * 2 + 1) * C + c] = S;
    } else if (last) {
        *st = S;
    }
}

// a, b: float [T, C] (acv_block_gates); seg_seq, seg_idx: the step's items (null: one item for each request, its whole
// portion); seg: float [items][2][C] scratch of the first launch, which runs when `summaries` is set.
ACV_API int acv_gated_scan(const float* a, const float* b, const void* y, int ldy, const float* yb, float* state,
                           const int* slots, const int* cu_q, const int* seg_seq, const int* seg_idx, int seg_len,
                           float* seg, int summaries, void* out, int ldo, int n_items, int C, int y_dtype, int dtype,
                           cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (C <= 0 || seg_len <= 0 || (summaries && (!seg || !seg_seq || !seg_idx))) return ACV_ERR_SIZE;
    dim3 grid(n_items, (C + 63) / 64);
#define SCAN_LAUNCH(TY, T)                                                                                           \
    {                                                                                                                \
        if (summaries) {                                                                                             \
            acv_launch(PDL_MISC, gated_scan_kernel<TY, T, true>, grid, 64, 0, stream, a, b, (const TY*)y, ldy, yb, state, \
                       slots, cu_q, seg_seq, seg_idx, seg_len, seg, (T*)out, ldo, C);                               \
            acv_launch(PDL_MISC, scan_fold_kernel, grid, 64, 0, stream, seg, seg_seq, seg_idx, seg_len, cu_q, C);    \
        }                                                                                                            \
        acv_launch(PDL_MISC, gated_scan_kernel<TY, T, false>, grid, 64, 0, stream, a, b, (const TY*)y, ldy, yb, state,    \
                   slots, cu_q, seg_seq, seg_idx, seg_len, seg, (T*)out, ldo, C);                                   \
        return acv_launch_status();                                                                                  \
    }
    if (y_dtype == ACV_F32 && dtype == ACV_F32) SCAN_LAUNCH(float, float)
    if (y_dtype == ACV_F32 && dtype == ACV_BF16) SCAN_LAUNCH(float, bf16)
    if (y_dtype == ACV_BF16 && dtype == ACV_BF16) SCAN_LAUNCH(bf16, bf16)
#undef SCAN_LAUNCH
    return ACV_ERR_DTYPE;
}
