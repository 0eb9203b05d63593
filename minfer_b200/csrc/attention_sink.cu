// Attention whose scores are changed before the softmax and whose softmax has a sink.
//
// For query head h (key/value head h / (n_heads / n_kv)), a query at position i and a key at
// position j:
//     s_ij = (q_i . k_j) * scale - r1[h] * ln(1 + r2[h] * (i - j))        (r1 == nullptr: no bias)
//     j is visible from i  iff  j <= i
//                          and  i - j < window                 (window > 0)
//                          and  floor(i / chunk) == floor(j / chunk)   (chunk > 0; counted from
//                                                               position 0 of the sequence)
//     w_ij = exp(s_ij) / (sink + sum over visible j' of exp(s_ij'))       (sink is 0 or 1: a key
//                                                               of score 0 that has no value)
//     o_i = sum_j w_ij v_j
// Keys have `hd` elements a head, values `vd`; the two differ freely.  Scores, the bias, the
// running maximum and sum, and the weighted sum are float32.
//
// Kernels here:
//   * unit_norm_kvstore: a fused q|k|v projection's float32 output (or its K splits) ->
//     q and k divided by their root mean square per head (no weight), v as it is; written
//     as the step's packed q, k, v and into the paged cache.
//   * sink_attention_generic: any sizes, float32 or bfloat16, keys from the step's packed
//     rows (whole prompts) or from the paged cache; one warp per (query, head).
//   * sink_attention_group (further down): bfloat16 on tensor cores.
#include "common.cuh"

#define SA_WARPS 4
#define SA_MAX_D 256

// ------------------------------------------------------------------------------------------
// q and k to unit root mean square per head, cache write
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(SA_WARPS * 32)
unit_norm_kvstore_kernel(const float* __restrict__ qkv, int n_partials, int n_tokens,
                         const int* __restrict__ positions, const int* __restrict__ token_row,
                         const int* __restrict__ seq_end, T* __restrict__ q_out,
                         T* __restrict__ k_out, T* __restrict__ v_out, T* __restrict__ k_cache,
                         T* __restrict__ v_cache, const int* __restrict__ page_table,
                         int table_stride, int ring, int n_heads, int n_kv, int hd, int vd,
                         float eps, int norm_qk, unsigned* __restrict__ status) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int b = token_row[t];
    // where this token's keys and values go in the cache: page and place in the page
    int page = -1;
    if (k_cache != nullptr) {
        bool keep = true;
        int p_eff = pos;
        if (ring > 0) {
            keep = pos >= seq_end[b] - ring;
            p_eff = pos % ring;
        }
        if (keep) {
            page = page_table[(size_t)b * table_stride + (p_eff >> 6)];
            if (page < 0 && threadIdx.x == 0 && blockIdx.y == 0)
                atomicOr(status, MF_STATUS_BAD_POSITION);
        }
    }
    pdl_wait();
    const size_t in_width = (size_t)(n_heads + n_kv) * hd + (size_t)n_kv * vd;
    const float* in = qkv + (size_t)t * in_width;
    const size_t plane = (size_t)n_tokens * in_width;
    const int n_items = n_heads + 2 * n_kv;
    // a warp takes a head: q heads, then k heads, then v heads
    for (int item = blockIdx.y * SA_WARPS + warp; item < n_items; item += gridDim.y * SA_WARPS) {
        const bool is_q = item < n_heads, is_v = item >= n_heads + n_kv;
        const int width = is_v ? vd : hd;
        const int hk = is_v ? item - n_heads - n_kv : item - n_heads;
        const size_t col0 = is_q ? (size_t)item * hd
                                 : (is_v ? (size_t)(n_heads + n_kv) * hd + (size_t)hk * vd
                                         : (size_t)(n_heads + hk) * hd);
        float val[SA_MAX_D / 32];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < SA_MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            float v = 0.0f;
            if (d < width) {
                v = in[col0 + d];
                for (int sp = 1; sp < n_partials; ++sp) v += in[sp * plane + col0 + d];
            }
            val[i] = v;
            ss = fmaf(v, v, ss);
        }
        float f = 1.0f;
        if (!is_v && norm_qk) {
            ss = warp_sum(ss);
            f = 1.0f / sqrtf(ss / (float)width + eps);
        }
        T* dst0 = nullptr;
        T* dst1 = nullptr;
        if (is_q) {
            dst0 = q_out + ((size_t)t * n_heads + item) * hd;
        } else {
            T* step_out = is_v ? v_out : k_out;
            if (step_out != nullptr) dst0 = step_out + ((size_t)t * n_kv + hk) * width;
            if (page >= 0)
                dst1 = (is_v ? v_cache : k_cache) +
                       (((size_t)page * n_kv + hk) * MF_PAGE + (pos & (MF_PAGE - 1))) * width;
        }
#pragma unroll
        for (int i = 0; i < SA_MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < width) {
                const T y = from_f32<T>(val[i] * f);
                if (dst0) dst0[d] = y;
                if (dst1) dst1[d] = y;
            }
        }
    }
}

extern "C" int mf_unit_norm_kvstore(const float* qkv, int n_partials, const int* positions,
                                    const int* token_row, const int* seq_end, void* q_out,
                                    void* k_out, void* v_out, void* k_cache, void* v_cache,
                                    const int* page_table, int table_stride, int ring,
                                    int n_tokens, int n_heads, int n_kv, int hd, int vd, float eps,
                                    int norm_qk, int dtype, unsigned* status,
                                    cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd < 1 || hd > SA_MAX_D || vd < 1 || vd > SA_MAX_D || n_partials < 0) return MF_ERR_UNSUPPORTED;
    if ((k_cache == nullptr) != (v_cache == nullptr)) return MF_ERR_ARGUMENT;
    if (k_cache != nullptr && page_table == nullptr) return MF_ERR_ARGUMENT;
    const int n_items = n_heads + 2 * n_kv;
    int by = 1;
    if (n_tokens < 2 * mf_sm_count()) {                  // few tokens: spread a token's heads
        by = (n_items + SA_WARPS - 1) / SA_WARPS;
        if (by > 16) by = 16;
    }
    dim3 grid(n_tokens, by);
#define MF_UNK(T) \
    mf_launch(unit_norm_kvstore_kernel<T>, grid, dim3(SA_WARPS * 32), 0, stream, qkv, n_partials, \
              n_tokens, positions, token_row, seq_end, (T*)q_out, (T*)k_out, (T*)v_out, \
              (T*)k_cache, (T*)v_cache, page_table, table_stride, ring, n_heads, n_kv, hd, vd, eps, \
              norm_qk, status)
    if (dtype == MF_DTYPE_F32) MF_UNK(float);
    else if (dtype == MF_DTYPE_BF16) MF_UNK(__nv_bfloat16);
    else return MF_ERR_UNSUPPORTED;
#undef MF_UNK
    return MF_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// the generic kernel: one warp per (query, head)
// ------------------------------------------------------------------------------------------
struct SinkArgs {
    const void* q;            // [rows][n_heads][hd]
    const void* k;            // packed keys [tokens][n_kv][hd]      (PAGED: [pages][n_kv][64][hd])
    const void* v;            // packed values [tokens][n_kv][vd]    (PAGED: [pages][n_kv][64][vd])
    const int* row_seq;       // [rows] batch row of each query
    const int* row_pos;       // [rows] absolute position of each query
    const int* cu_seqlens;    // [B+1] packed source only
    const int* page_table;    // paged source only
    int table_stride;
    int ring;                 // paged source: 0 = linear, else ring length in positions
    void* out;                // [rows][n_heads * vd]
    const float* r1;          // [n_heads] or nullptr
    const float* r2;          // [n_heads]
    int rows, n_heads, n_kv, hd, vd;
    int window, chunk, sink;
    float scale;
};

// first visible key of a query at `pos`
__device__ __forceinline__ int sink_first_key(int pos, int window, int chunk) {
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    return lo;
}

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// VEC: hd is a multiple of the 16-byte vector (rows of keys then start on 16-byte boundaries)
template <typename T, bool PAGED, bool VEC>
__global__ void __launch_bounds__(SA_WARPS * 32) sink_attention_generic_kernel(SinkArgs a) {
    pdl_launch_dependents();
    __shared__ float q_s[SA_WARPS][SA_MAX_D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long item = (long long)blockIdx.x * SA_WARPS + warp;
    if (item >= (long long)a.rows * a.n_heads) return;      // no block-wide barrier below
    const int head = (int)(item % a.n_heads);
    const int row = (int)(item / a.n_heads);
    const int hd = a.hd, vd = a.vd;
    const int hk = head / (a.n_heads / a.n_kv);
    const int b = a.row_seq[row];
    const int pos = a.row_pos[row];
    const int lo = sink_first_key(pos, a.window, a.chunk);
    const int hi = pos + 1;
    const float r1 = a.r1 ? a.r1[head] : 0.0f;
    const float r2 = a.r1 ? a.r2[head] : 0.0f;
    const long long packed0 = PAGED ? 0 : (long long)a.cu_seqlens[b];
    pdl_wait();

    const T* q = (const T*)a.q + ((size_t)row * a.n_heads + head) * hd;
    for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32(q[d]) * a.scale;
    __syncwarp();

    const T* kbase = (const T*)a.k;
    const T* vbase = (const T*)a.v;
    // the sink is a key of score 0 without a value: it starts the running maximum and sum
    float m = a.sink ? 0.0f : -INFINITY, l = a.sink ? 1.0f : 0.0f;
    float acc[SA_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < SA_MAX_D / 32; ++i) acc[i] = 0.0f;

    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < hi;
        long long krow = 0;                           // index of key j's row: [..][hk][j]
        if (valid) {
            if (PAGED) {
                const int p_eff = a.ring > 0 ? j % a.ring : j;
                const int page = a.page_table[(size_t)b * a.table_stride + (p_eff >> 6)];
                krow = ((long long)page * a.n_kv + hk) * MF_PAGE + (j & (MF_PAGE - 1));
            } else {
                krow = (packed0 + j) * a.n_kv + hk;
            }
        }
        float s = -INFINITY;
        if (valid) {
            const T* kr = kbase + krow * hd;
            float dot = 0.0f;
            if (VEC) {
                for (int d = 0; d < hd; d += Vec16<T>::N) {
                    float kv[Vec16<T>::N];
                    Vec16<T>::load(kr + d, kv);
#pragma unroll
                    for (int e = 0; e < Vec16<T>::N; ++e) dot = fmaf(q_s[warp][d + e], kv[e], dot);
                }
            } else {
                for (int d = 0; d < hd; ++d) dot = fmaf(q_s[warp][d], to_f32(kr[d]), dot);
            }
            s = dot;
            if (a.r1) s -= r1 * log1pf(r2 * (float)(pos - j));
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);           // 0 on the first tile without a sink
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < SA_MAX_D / 32; ++i) acc[i] *= corr;
        const int n_here = min(32, hi - j0);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long vrow = __shfl_sync(0xffffffffu, krow, jj);
            const T* vr = vbase + vrow * vd;
#pragma unroll
            for (int i = 0; i < SA_MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
    T* o = (T*)a.out + ((size_t)row * a.n_heads + head) * vd;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < SA_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) o[d] = from_f32<T>(acc[i] * inv);
    }
}

static int sink_check(const SinkArgs& a, int dtype) {
    if (dtype != MF_DTYPE_F32 && dtype != MF_DTYPE_BF16) return MF_ERR_UNSUPPORTED;
    if (a.hd < 1 || a.hd > SA_MAX_D || a.vd < 1 || a.vd > SA_MAX_D) return MF_ERR_UNSUPPORTED;
    if (a.n_kv < 1 || a.n_heads % a.n_kv != 0) return MF_ERR_ARGUMENT;
    if (a.window < 0 || a.chunk < 0) return MF_ERR_ARGUMENT;
    return 0;
}

template <bool PAGED>
static int sink_generic_launch(const SinkArgs& a, int dtype, cudaStream_t stream) {
    if (a.rows <= 0) return 0;
    const long long items = (long long)a.rows * a.n_heads;
    dim3 grid((unsigned)((items + SA_WARPS - 1) / SA_WARPS)), block(SA_WARPS * 32);
    if (dtype == MF_DTYPE_F32) {
        if (a.hd % 4 == 0) mf_launch(sink_attention_generic_kernel<float, PAGED, true>, grid, block, 0, stream, a);
        else mf_launch(sink_attention_generic_kernel<float, PAGED, false>, grid, block, 0, stream, a);
    } else {
        if (a.hd % 8 == 0) mf_launch(sink_attention_generic_kernel<__nv_bfloat16, PAGED, true>, grid, block, 0, stream, a);
        else mf_launch(sink_attention_generic_kernel<__nv_bfloat16, PAGED, false>, grid, block, 0, stream, a);
    }
    return MF_LAUNCH_CHECK();
}

static SinkArgs sink_args(const void* q, const void* k, const void* v, const int* row_seq,
                          const int* row_pos, const int* cu_seqlens, const int* page_table,
                          int table_stride, int ring, void* out, const float* r1, const float* r2,
                          int rows, int n_heads, int n_kv, int hd, int vd, int window, int chunk,
                          int sink, float scale) {
    SinkArgs a;
    a.q = q; a.k = k; a.v = v; a.row_seq = row_seq; a.row_pos = row_pos; a.cu_seqlens = cu_seqlens;
    a.page_table = page_table; a.table_stride = table_stride; a.ring = ring; a.out = out;
    a.r1 = r1; a.r2 = r2; a.rows = rows; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.vd = vd;
    a.window = window; a.chunk = chunk; a.sink = sink ? 1 : 0; a.scale = scale;
    return a;
}

// keys and values are the step's own packed rows: position j of batch row b lies at token
// cu_seqlens[b] + j (whole prompts)
extern "C" int mf_sink_attention_packed(const void* q, const void* k, const void* v,
                                        const int* row_seq, const int* row_pos,
                                        const int* cu_seqlens, void* out, const float* r1,
                                        const float* r2, int rows, int n_heads, int n_kv, int hd,
                                        int vd, int window, int chunk, int sink, float scale,
                                        int dtype, cudaStream_t stream) {
    SinkArgs a = sink_args(q, k, v, row_seq, row_pos, cu_seqlens, nullptr, 0, 0, out, r1, r2, rows,
                           n_heads, n_kv, hd, vd, window, chunk, sink, scale);
    const int bad = sink_check(a, dtype);
    if (bad) return bad;
    return sink_generic_launch<false>(a, dtype, stream);
}

// keys and values come from the paged cache, the step's own among them
extern "C" int mf_sink_attention_paged(const void* q, const void* k_cache, const void* v_cache,
                                       const int* row_seq, const int* row_pos,
                                       const int* page_table, int table_stride, int ring,
                                       void* out, const float* r1, const float* r2, int rows,
                                       int n_heads, int n_kv, int hd, int vd, int window,
                                       int chunk, int sink, float scale, int dtype,
                                       cudaStream_t stream) {
    SinkArgs a = sink_args(q, k_cache, v_cache, row_seq, row_pos, nullptr, page_table,
                           table_stride, ring, out, r1, r2, rows, n_heads, n_kv, hd, vd, window,
                           chunk, sink, scale);
    const int bad = sink_check(a, dtype);
    if (bad) return bad;
    if (page_table == nullptr) return MF_ERR_ARGUMENT;
    return sink_generic_launch<true>(a, dtype, stream);
}
