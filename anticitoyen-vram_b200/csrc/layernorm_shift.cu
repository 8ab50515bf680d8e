// Layer norm over a float residual stream, and the token shift of a mixer's input.
//
//   x += delta_scale * delta                       (float; delta has the run's element type; written back)
//   n  = (x - mean) / sqrt(var + eps) * w + b      var = mean of the squared deviations, two passes over the row
//
//   token shift:  h'[t] = n[t] + (n[t-1] - n[t]) * mu[c]
//
// where n[t-1] is the normed row of the request's previous token: the row before in the step, or, for the
// first token that a request brings to a step, the row that the request's state slot keeps from its last step
// (zeros when the request begins: the slot is zeroed at admission).  The slot then takes the normed row of the
// request's last token of this step.
//
// Three kernels:
//   * acv_add_layernorm        x (+= delta) -> norm, as element type T or as float; optionally only some rows
//   * acv_token_shift          float normed rows -> shifted rows of type T, state read and replaced
//   * acv_add_layernorm_shift  both in one launch for steps in which every request brings one token
// In acv_token_shift the block of a request's first token is the one that replaces the state, after it has read
// it, element by element in the same thread: no other block touches that slot.
#include "common.cuh"

template <typename TD, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, float delta_scale,
                                     const float* __restrict__ w, const float* __restrict__ b, TO* __restrict__ out,
                                     const int* __restrict__ rows, int H, float eps) {
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    float* xr = x + (size_t)r_in * H;
    const TD* dr = delta ? delta + (size_t)r_in * H : nullptr;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (dr) {
            v = fmaf(delta_scale, to_f32(dr[i]), v);
            if (!rows) xr[i] = v;
        }
        row[i] = v;
        s += v;
    }
    const float mean = block_sum(s, red) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row[i] - mean;
        ss += d * d;
    }
    const float rs = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps);
    TO* o = out + (size_t)r_out * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>(fmaf((row[i] - mean) * rs, w[i], b ? b[i] : 0.f));
}

template <typename TO>
__global__ void token_shift_kernel(const float* __restrict__ n, const float* __restrict__ mu, float* __restrict__ state,
                                   const int* __restrict__ slots, const int* __restrict__ cu_q,
                                   const int* __restrict__ seq_of_token, TO* __restrict__ out, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    const int first = cu_q[seq], last = cu_q[seq + 1] - 1;
    const float* cur = n + (size_t)t * H;
    TO* o = out + (size_t)t * H;
    if (t != first) {
        const float* prev = cur - H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>(fmaf(prev[i] - cur[i], mu[i], cur[i]));
        return;
    }
    float* st = state + (size_t)slots[seq] * H;
    const float* keep = n + (size_t)last * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float prev = st[i];
        st[i] = keep[i];
        o[i] = from_f32<TO>(fmaf(prev - cur[i], mu[i], cur[i]));
    }
}

// every request of the step brings one token: row t is request t
template <typename TD, typename TO>
__global__ void add_layernorm_shift_kernel(float* __restrict__ x, const TD* __restrict__ delta, float delta_scale,
                                           const float* __restrict__ w, const float* __restrict__ b,
                                           const float* __restrict__ mu, float* __restrict__ state,
                                           const int* __restrict__ slots, TO* __restrict__ out, int H, float eps) {
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    float* xr = x + (size_t)t * H;
    const TD* dr = delta ? delta + (size_t)t * H : nullptr;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (dr) {
            v = fmaf(delta_scale, to_f32(dr[i]), v);
            xr[i] = v;
        }
        row[i] = v;
        s += v;
    }
    const float mean = block_sum(s, red) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row[i] - mean;
        ss += d * d;
    }
    const float rs = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps);
    float* st = state + (size_t)slots[t] * H;
    TO* o = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float cur = fmaf((row[i] - mean) * rs, w[i], b ? b[i] : 0.f);
        const float prev = st[i];
        st[i] = cur;
        o[i] = from_f32<TO>(fmaf(prev - cur, mu[i], cur));
    }
}

static inline int ln_threads(int H) { return H >= 4096 ? 512 : (H >= 1024 ? 256 : 128); }

template <typename Kernel>
static int ln_smem(Kernel kernel, size_t smem) {
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    if (smem > 48 * 1024) {
        static AcvSmemConfig cfg;
        return acv_ensure_smem(cfg, kernel, (int)smem);
    }
    return 0;
}

// delta_dtype: element type of delta; out_dtype: of out (float output serves the token shift's first pass)
ACV_API int acv_add_layernorm(float* x, const void* delta, float delta_scale, const float* w, const float* b, void* out,
                              const int* rows, int n_rows, int H, float eps, int delta_dtype, int out_dtype,
                              cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    const int threads = ln_threads(H);
#define LN_CASE(TD, TO)                                                                                              \
    {                                                                                                                \
        const int e = ln_smem(add_layernorm_kernel<TD, TO>, smem);                                                   \
        if (e) return e;                                                                                             \
        acv_launch(PDL_NORM, add_layernorm_kernel<TD, TO>, n_rows, threads, smem, stream, x, (const TD*)delta,       \
                   delta_scale, w, b, (TO*)out, rows, H, eps);                                                       \
        return acv_launch_status();                                                                                  \
    }
    if (delta_dtype == ACV_F32 && out_dtype == ACV_F32) LN_CASE(float, float)
    if (delta_dtype == ACV_BF16 && out_dtype == ACV_F32) LN_CASE(bf16, float)
    if (delta_dtype == ACV_BF16 && out_dtype == ACV_BF16) LN_CASE(bf16, bf16)
    if (delta_dtype == ACV_F32 && out_dtype == ACV_BF16) LN_CASE(float, bf16)
#undef LN_CASE
    return ACV_ERR_DTYPE;
}

ACV_API int acv_token_shift(const float* n, const float* mu, float* state, const int* slots, const int* cu_q,
                            const int* seq_of_token, void* out, int T, int H, int out_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = ln_threads(H);
    if (out_dtype == ACV_F32)
        acv_launch(PDL_NORM, token_shift_kernel<float>, T, threads, 0, stream, n, mu, state, slots, cu_q, seq_of_token,
                   (float*)out, H);
    else if (out_dtype == ACV_BF16)
        acv_launch(PDL_NORM, token_shift_kernel<bf16>, T, threads, 0, stream, n, mu, state, slots, cu_q, seq_of_token,
                   (bf16*)out, H);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

ACV_API int acv_add_layernorm_shift(float* x, const void* delta, float delta_scale, const float* w, const float* b,
                                    const float* mu, float* state, const int* slots, void* out, int T, int H, float eps,
                                    int delta_dtype, int out_dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    const int threads = ln_threads(H);
#define LNS_CASE(TD, TO)                                                                                             \
    {                                                                                                                \
        const int e = ln_smem(add_layernorm_shift_kernel<TD, TO>, smem);                                             \
        if (e) return e;                                                                                             \
        acv_launch(PDL_NORM, add_layernorm_shift_kernel<TD, TO>, T, threads, smem, stream, x, (const TD*)delta,      \
                   delta_scale, w, b, mu, state, slots, (TO*)out, H, eps);                                           \
        return acv_launch_status();                                                                                  \
    }
    if (delta_dtype == ACV_F32 && out_dtype == ACV_F32) LNS_CASE(float, float)
    if (delta_dtype == ACV_BF16 && out_dtype == ACV_BF16) LNS_CASE(bf16, bf16)
#undef LNS_CASE
    return ACV_ERR_DTYPE;
}

// x[t][c] += v[c] over a float stream (a vector that joins the stream between two layers)
__global__ void add_row_f32_kernel(float* __restrict__ x, const float* __restrict__ v, long long n, int H) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] += v[i % H];
}

ACV_API int acv_add_row_f32(float* x, const float* v, int T, int H, cudaStream_t stream) {
    const long long n = (long long)T * H;
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    acv_launch(PDL_MISC, add_row_f32_kernel, blocks, 256, 0, stream, x, v, n, H);
    return acv_launch_status();
}

// logits <- cap * tanh(logits / cap), in place, float
__global__ void softcap_f32_kernel(float* __restrict__ x, size_t n, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

ACV_API int acv_softcap_f32(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return ACV_ERR_SIZE;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    acv_launch(PDL_MISC, softcap_f32_kernel, blocks, 256, 0, stream, x, (size_t)n, cap);
    return acv_launch_status();
}
