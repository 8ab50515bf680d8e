// Differential attention over the paged cache: two attention maps per head that share one set of values.
//
// A query head holds two query vectors of D elements, [map 1 | map 2]; a key/value head holds two key
// vectors laid out the same way (a key row of 2*D elements in the pages) and one value vector of DV
// elements.  For a query at absolute position p and the keys j it may see:
//
//     s_a[j] = scale * <q_a, k_a[j]>            a = 1, 2        (32-bit)
//     o_a    = sum_j softmax(s_a)[j] * v[j]                     (each map its own softmax, same values)
//     o      = o_1 - lambda * o_2
//     out    = o / sqrt(mean(o^2) + eps) * out_scale            (over the DV values of the head, no weight)
//
// lambda and out_scale are numbers of the layer that the caller folds from its weights and constants.
// Which keys a query sees is a parameter: j <= p always; with window > 0 only j > p - window; with
// chunk > 0 only the keys of the query's own chunk, floor(j / chunk) == floor(p / chunk), chunks being
// counted from position 0 of the request whatever portion of it the step brings.
//
// Two kernels share this file:
//   * acv_heads_norm_append: per-vector RMS norm (weight shared by all heads and maps) of the projected
//     queries (in place) and keys (into their pages), and the copy of the values into theirs.  Key rows
//     and value rows may differ in size, so keys and values have page tensors of their own shape.
//   * acv_diff_attention_generic: one warp per (token, query head), any sizes, float or bfloat16: the
//     32-bit path, and the fallback of the bfloat16 path for sizes that the tensor-core kernels refuse.
#include "common.cuh"

#define DA_WARPS 4

// ----------------------------------------------------------------------------- norm of the heads' vectors + append
// q: [T, NQ vectors of D], k: [T, NK vectors of D] (NK / NKV vectors make one key row), v: [T, NKV rows of DV].
// One warp per vector (q, k) or value row.  Null k skips keys and values (a layer that reads another layer's).
// With q_out the normed query vectors do not go back in place: vector a of a head (a < per = NK / NKV) becomes a query
// row of its own, per * D elements long, that holds the vector at offset a * D and zeros elsewhere.  Such a row's
// product with a whole key row is the map's score, so attention kernels that know one query vector per head serve
// the maps as 'per' times as many heads over the same key/value heads.
template <typename T>
__global__ void heads_norm_append_kernel(T* __restrict__ q, T* __restrict__ q_out, int q_out_stride, const T* __restrict__ k,
                                         const T* __restrict__ v, int row_stride,
                                         int NQ, int NK, int NKV, int D, int DV, const float* __restrict__ q_w,
                                         const float* __restrict__ k_w, float eps, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                         int bt_stride, const int* __restrict__ bt_rows, T* __restrict__ k_pages,
                                         T* __restrict__ v_pages, int page_size, int num_pages) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.y * DA_WARPS + warp;
    const int t = blockIdx.x;
    const int units = NQ + (k ? NK + NKV : 0);
    if (unit >= units) return;
    const bool is_q = unit < NQ;
    const bool is_k = !is_q && unit < NQ + NK;
    long long page_row = -1;
    if (!is_q) {
        const int pos = positions[t];
        const int seq = seq_of_token[t];
        const int pg = block_table[(size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride + pos / page_size];
        if (pg < 0 || pg >= num_pages) return;      // a padding row of a fixed-shape batch keeps nothing
        page_row = (long long)pg * NKV * page_size + (pos % page_size);
    }
    if (!is_q && !is_k) {
        const int kvh = unit - NQ - NK;
        const T* src = v + (size_t)t * row_stride + (size_t)kvh * DV;
        T* dst = v_pages + (page_row + (long long)kvh * page_size) * DV;
        for (int e = lane; e < DV; e += 32) dst[e] = src[e];
        return;
    }
    const int vec = is_q ? unit : unit - NQ;
    const T* src = (is_q ? q : k) + (size_t)t * row_stride + (size_t)vec * D;
    const float* w = is_q ? q_w : k_w;
    float ss = 0.f;
    for (int e = lane; e < D; e += 32) {
        const float x = to_f32(src[e]);
        ss += x * x;
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    T* dst;
    if (is_q && q_out) {
        const int per = NK / NKV;
        T* wide = q_out + (size_t)t * q_out_stride + (size_t)vec * per * D;
        const int a = vec % per;
        for (int e = lane; e < per * D; e += 32)
            if (e / D != a) wide[e] = from_f32<T>(0.f);
        dst = wide + a * D;
    } else if (is_q) {
        dst = q + (size_t)t * row_stride + (size_t)vec * D;
    } else {
        const int per = NK / NKV;                   // key vectors in one key row
        const int kvh = vec / per, a = vec - kvh * per;
        dst = k_pages + (page_row + (long long)kvh * page_size) * ((long long)per * D) + (long long)a * D;
    }
    for (int e = lane; e < D; e += 32) dst[e] = from_f32<T>(to_f32(src[e]) * inv * (w ? w[e] : 1.f));
}

ACV_API int acv_heads_norm_append(void* q, void* q_out, int q_out_stride, const void* k, const void* v, int row_stride, int T_tokens, int NQ, int NK, int NKV,
                                  int D, int DV, const float* q_w, const float* k_w, float eps, const int* positions,
                                  const int* seq_of_token, const int* block_table, int bt_stride, const int* bt_rows,
                                  void* k_pages, void* v_pages, int page_size, int num_pages, int dtype, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (q_out && (NKV <= 0 || NK <= 0 || NK % NKV)) return ACV_ERR_SIZE;
    if (D <= 0 || NQ <= 0 || (k && (NKV <= 0 || NK % NKV || DV <= 0 || !v || !k_pages || !v_pages || !block_table)))
        return ACV_ERR_SIZE;
    const int units = NQ + (k ? NK + NKV : 0);
    dim3 grid(T_tokens, (units + DA_WARPS - 1) / DA_WARPS);
    if (dtype == ACV_F32)
        acv_launch(PDL_ROPE, heads_norm_append_kernel<float>, grid, DA_WARPS * 32, 0, stream, (float*)q, (float*)q_out, q_out_stride,
                   (const float*)k, (const float*)v, row_stride, NQ, NK, NKV, D, DV, q_w, k_w, eps, positions, seq_of_token, block_table,
                   bt_stride, bt_rows, (float*)k_pages, (float*)v_pages, page_size, num_pages);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_ROPE, heads_norm_append_kernel<bf16>, grid, DA_WARPS * 32, 0, stream, (bf16*)q, (bf16*)q_out, q_out_stride,
                   (const bf16*)k, (const bf16*)v, row_stride, NQ, NK, NKV, D, DV, q_w, k_w, eps, positions, seq_of_token, block_table,
                   bt_stride, bt_rows, (bf16*)k_pages, (bf16*)v_pages, page_size, num_pages);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- generic form
// One warp per (token, query head).  The two query vectors wait in shared memory as floats, scaled; a lane
// takes one key of a tile of 32 and computes both scores; each map keeps a running maximum and sum of its
// own, and both accumulate the same value rows.  NR = ceil(DV / 32) accumulator registers per map.
template <typename T, int NR>
__global__ void diff_attn_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                         const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                         const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows,
                                         int NH, int NKV, int D, int DV, int page_size, int num_pages, float scale, int window,
                                         int chunk, float lambda, float eps, float out_scale) {
    extern __shared__ float sm_all[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * DA_WARPS + warp;
    const int t = blockIdx.x;
    if (h >= NH) return;
    const int KD = 2 * D;
    float* qs = sm_all + warp * KD;
    const int kvh = h / (NH / NKV);
    const int p = positions[t];
    const int seq = seq_of_token[t];
    const int* bt = block_table + (size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * KD;
    for (int e = lane; e < KD; e += 32) qs[e] = to_f32(qrow[e]) * scale;
    __syncwarp();

    float acc1[NR], acc2[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc1[r] = acc2[r] = 0.f;
    float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
    int lo = chunk > 0 ? (p / chunk) * chunk : 0;
    if (window > 0) lo = max(lo, p - window + 1);

    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        bool valid = j <= p;
        long long row = 0;
        if (valid) {
            const int pg = bt[j / page_size];
            valid = pg >= 0 && pg < num_pages;
            row = ((long long)pg * NKV + kvh) * page_size + (j % page_size);
        }
        float s1 = -INFINITY, s2 = -INFINITY;
        if (valid) {
            const T* kr = k_pages + row * KD;
            float d1 = 0.f, d2 = 0.f;
            for (int e = 0; e < D; ++e) {
                d1 = fmaf(qs[e], to_f32(kr[e]), d1);
                d2 = fmaf(qs[D + e], to_f32(kr[D + e]), d2);
            }
            s1 = d1;
            s2 = d2;
        }
        const float t1 = warp_max(s1), t2 = warp_max(s2);
        if (t1 == -INFINITY) continue;   // uniform: no readable key in this tile (both maps see the same keys)
        const float n1 = fmaxf(m1, t1), n2 = fmaxf(m2, t2);
        const float a1 = expf(m1 - n1), a2 = expf(m2 - n2);
        const float p1 = valid ? expf(s1 - n1) : 0.f, p2 = valid ? expf(s2 - n2) : 0.f;
        l1 = l1 * a1 + warp_sum(p1);
        l2 = l2 * a2 + warp_sum(p2);
        m1 = n1;
        m2 = n2;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            acc1[r] *= a1;
            acc2[r] *= a2;
        }
        const int n_in_tile = min(32, p - j0 + 1);
        for (int kk = 0; kk < n_in_tile; ++kk) {
            const float w1 = __shfl_sync(0xffffffffu, p1, kk), w2 = __shfl_sync(0xffffffffu, p2, kk);
            const long long ro = __shfl_sync(0xffffffffu, row, kk);
            if (w1 == 0.f && w2 == 0.f) continue;
            const T* vr = v_pages + ro * DV;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int e = lane + 32 * r;
                if (e < DV) {
                    const float x = to_f32(vr[e]);
                    acc1[r] = fmaf(w1, x, acc1[r]);
                    acc2[r] = fmaf(w2, x, acc2[r]);
                }
            }
        }
    }
    const float i1 = l1 > 0.f ? 1.f / l1 : 0.f, i2 = l2 > 0.f ? 1.f / l2 : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        acc1[r] = acc1[r] * i1 - lambda * (acc2[r] * i2);
        if (lane + 32 * r < DV) ss += acc1[r] * acc1[r];
    }
    ss = warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)DV + eps);
    T* orow = out + (size_t)t * out_stride + (size_t)h * DV;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int e = lane + 32 * r;
        if (e < DV) orow[e] = from_f32<T>(acc1[r] * f);
    }
}

template <typename T>
static int launch_diff_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                               const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                               const int* bt_rows, int T_tokens, int NH, int NKV, int D, int DV, int page_size, int num_pages,
                               float scale, int window, int chunk, float lambda, float eps, float out_scale, cudaStream_t stream) {
    dim3 grid(T_tokens, (NH + DA_WARPS - 1) / DA_WARPS);
    const size_t smem = (size_t)DA_WARPS * 2 * D * sizeof(float);
    const int nr = (DV + 31) / 32;
#define DA_CASE(N)                                                                                                      \
    case N:                                                                                                             \
        acv_launch(PDL_ATTN, diff_attn_generic_kernel<T, N>, grid, DA_WARPS * 32, smem, stream, (const T*)q, q_stride,  \
                   (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages, positions, seq_of_token, block_table,     \
                   bt_stride, bt_rows, NH, NKV, D, DV, page_size, num_pages, scale, window, chunk, lambda, eps, out_scale); \
        break;
    switch (nr) {
        DA_CASE(1) DA_CASE(2) DA_CASE(3) DA_CASE(4) DA_CASE(5) DA_CASE(6) DA_CASE(7) DA_CASE(8)
        default: return ACV_ERR_SIZE;
    }
#undef DA_CASE
    return acv_launch_status();
}

ACV_API int acv_diff_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                       const void* v_pages, const int* positions, const int* seq_of_token,
                                       const int* block_table, int bt_stride, const int* bt_rows, int T_tokens, int NH, int NKV,
                                       int D, int DV, int page_size, int num_pages, float scale, int window, int chunk,
                                       float lambda, float eps, float out_scale, int dtype, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (D <= 0 || D > 1024 || DV <= 0 || DV > 256 || NKV <= 0 || NH % NKV) return ACV_ERR_SIZE;
    if (dtype == ACV_F32)
        return launch_diff_generic<float>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token, block_table,
                                          bt_stride, bt_rows, T_tokens, NH, NKV, D, DV, page_size, num_pages, scale, window, chunk,
                                          lambda, eps, out_scale, stream);
    if (dtype == ACV_BF16)
        return launch_diff_generic<bf16>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token, block_table,
                                         bt_stride, bt_rows, T_tokens, NH, NKV, D, DV, page_size, num_pages, scale, window, chunk,
                                         lambda, eps, out_scale, stream);
    return ACV_ERR_DTYPE;
}

// ----------------------------------------------------------------------------- the maps' outputs combined
// maps: [T, NH * 2 rows of DV] (head h's map 1, then its map 2, as attention kernels with one query vector per head
// leave them); out[t, h] = unit_rms(o1 - lambda o2) * out_scale, in 32-bit.  One warp per (token, head).
template <typename T, typename TM, int NR>
__global__ void diff_combine_kernel(const TM* __restrict__ maps, int maps_stride, T* __restrict__ out, int out_stride, int NH,
                                    int DV, float lambda, float eps, float out_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * DA_WARPS + warp;
    const int t = blockIdx.x;
    if (h >= NH) return;
    const TM* a1 = maps + (size_t)t * maps_stride + (size_t)(2 * h) * DV;
    const TM* a2 = a1 + DV;
    float o[NR];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int e = lane + 32 * r;
        o[r] = e < DV ? to_f32(a1[e]) - lambda * to_f32(a2[e]) : 0.f;
        ss += o[r] * o[r];
    }
    ss = warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)DV + eps);
    T* orow = out + (size_t)t * out_stride + (size_t)h * DV;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int e = lane + 32 * r;
        if (e < DV) orow[e] = from_f32<T>(o[r] * f);
    }
}

// maps_f32: the maps are float beside a bfloat16 output (they were never rounded: the difference of two nearly equal
// maps keeps its digits)
ACV_API int acv_diff_combine(const void* maps, int maps_stride, int maps_f32, void* out, int out_stride, int T_tokens, int NH,
                             int DV, float lambda, float eps, float out_scale, int dtype, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (DV <= 0 || DV > 256 || NH <= 0) return ACV_ERR_SIZE;
    dim3 grid(T_tokens, (NH + DA_WARPS - 1) / DA_WARPS);
    const int nr = (DV + 31) / 32;
#define DC_CASE(TT, TM, N)                                                                                              \
    case N:                                                                                                             \
        acv_launch(PDL_ATTN, diff_combine_kernel<TT, TM, N>, grid, DA_WARPS * 32, 0, stream, (const TM*)maps,           \
                   maps_stride, (TT*)out, out_stride, NH, DV, lambda, eps, out_scale);                                  \
        break;
#define DC_ALL(TT, TM) switch (nr) { DC_CASE(TT, TM, 1) DC_CASE(TT, TM, 2) DC_CASE(TT, TM, 3) DC_CASE(TT, TM, 4) \
                                     DC_CASE(TT, TM, 5) DC_CASE(TT, TM, 6) DC_CASE(TT, TM, 7) DC_CASE(TT, TM, 8) }
    if (dtype == ACV_F32) {
        DC_ALL(float, float)
    } else if (dtype == ACV_BF16 && maps_f32) {
        DC_ALL(bf16, float)
    } else if (dtype == ACV_BF16) {
        DC_ALL(bf16, bf16)
    } else {
        return ACV_ERR_DTYPE;
    }
#undef DC_ALL
#undef DC_CASE
    return acv_launch_status();
}
