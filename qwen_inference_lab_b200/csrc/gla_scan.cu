// Gated linear attention with a decay per key channel, as a scan over the tokens of every segment.
//
// Per head, with a state S [d, e] (d key channels, e value channels) kept in float32 per request:
//
//   a_t = sigmoid(z_t)^(1/tau),  z_t = A2 low_t + b           (float32; low_t is the low-rank projection)
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T
//   o_t = S_t^T (q_t * q_scale)
//   y_t = o_t / sqrt(mean_e(o_t^2) + eps) * w  *  silu(g_t)   (norm over the head's e values, gate from a projection)
//
// One block owns one (segment, head, tile of value columns): a thread holds a slice of one column of S in
// registers for the whole segment, reads the state slot of the segment's request at the start and writes
// it back at the end, so a prompt portion goes on from what the portions before it left, and a single
// decoded token is a segment of length one.  When one tile holds all of a head's value columns the norm
// and the gate are applied by the same block; otherwise o goes to a float32 scratch buffer and a row
// kernel norms and gates it.  Tokens are taken in their order with float32 arithmetic, so the
// result does not depend on how a sequence was cut into segments.  Tokens are staged in batches of
// GLA_TB: one barrier pair per batch instead of per token.
//
// q, k, v, g and low are column ranges of one row-major buffer (the stacked projection), given as
// pointers to their first column and the common row stride.
#include "common.cuh"

#define GLA_TB 8

__device__ __forceinline__ float decay_from_logit(float z, float inv_tau) {
    // sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau);  log_sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
    const float log_sigmoid = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
    return expf(log_sigmoid * inv_tau);
}

#define GLA_R 32          // rows of a column that one thread holds
#define GLA_THREADS 256

template <typename T, typename W>
__device__ __forceinline__ void gla_norm_gate_rows(const float* o_rows, int o_stride, int nb, size_t first_token,
                                                   const T* g, int ld, const W* norm_w, float eps, int n_heads,
                                                   int head, int e, T* out, int lane, int warp, int warps) {
    for (int tb = warp; tb < nb; tb += warps) {
        const float* o = o_rows + (size_t)tb * o_stride;
        float ss = 0.f;
        for (int c = lane; c < e; c += 32) ss = fmaf(o[c], o[c], ss);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)e + eps);
        const size_t token = first_token + tb;
        for (int c = lane; c < e; c += 32) {
            const float gate = to_f32<T>(g[token * ld + head * e + c]);
            const float y = o[c] * scale * to_f32<W>(norm_w[c]);
            out[(token * n_heads + head) * e + c] = from_f32<T>(y * (gate / (1.f + expf(-gate))));
        }
    }
}

template <typename T, typename W, bool FUSED>
__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                const T* __restrict__ low, int ld, const W* __restrict__ a2, const W* __restrict__ a2_bias, int rank,
                float inv_tau, float q_scale, const W* __restrict__ norm_w, float eps,
                float* __restrict__ state, const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                const int* __restrict__ seg_row, int n_heads, int d, int e, int ds_count, int tile_cols,
                float* __restrict__ o_raw, T* __restrict__ out) {
    constexpr int R = GLA_R;
    extern __shared__ float smem[];
    float* sq = smem;                    // [TB][d]
    float* sk = sq + GLA_TB * d;         // [TB][d]
    float* sa = sk + GLA_TB * d;         // [TB][d]
    float* sv = sa + GLA_TB * d;         // [TB][tile_cols]
    float* so = sv + GLA_TB * tile_cols; // [TB][tile_cols]
    qil_wait_for_producer();
    qil_release_consumer();
    const int tiles = (e + tile_cols - 1) / tile_cols;
    const int head = blockIdx.x / tiles, col0 = (blockIdx.x % tiles) * tile_cols, seg = blockIdx.y;
    const int first = seg_start[seg], count = seg_len[seg], row = seg_row[seg];
    const int tid = threadIdx.x, threads = blockDim.x;
    const int local = tid / ds_count, ds = tid % ds_count, col = col0 + local;
    const bool owner = local < tile_cols && col < e;
    float* slot = state + ((size_t)row * n_heads + head) * d * e;

    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int dd = r * ds_count + ds;
        S[r] = (owner && dd < d) ? slot[(size_t)dd * e + col] : 0.f;
    }
    const int lane = tid & 31, warp = tid >> 5, warps = threads >> 5;
    for (int t0 = 0; t0 < count; t0 += GLA_TB) {
        const int nb = count - t0 < GLA_TB ? count - t0 : GLA_TB;
        __syncthreads();
        for (int i = tid; i < nb * d; i += threads) {
            const int tb = i / d, dd = i % d;
            const size_t at = (size_t)(first + t0 + tb) * ld + head * d + dd;
            sq[tb * d + dd] = to_f32<T>(q[at]) * q_scale;
            sk[tb * d + dd] = to_f32<T>(k[at]);
            const int channel = head * d + dd;
            float z = to_f32<W>(a2_bias[channel]);
            const T* low_row = low + (size_t)(first + t0 + tb) * ld;
            const W* a2_row = a2 + (size_t)channel * rank;
            for (int j = 0; j < rank; ++j) z = fmaf(to_f32<W>(a2_row[j]), to_f32<T>(low_row[j]), z);
            sa[tb * d + dd] = decay_from_logit(z, inv_tau);
        }
        for (int i = tid; i < nb * tile_cols; i += threads) {
            const int tb = i / tile_cols, c = col0 + i % tile_cols;
            sv[i] = c < e ? to_f32<T>(v[(size_t)(first + t0 + tb) * ld + head * e + c]) : 0.f;
        }
        __syncthreads();
        for (int tb = 0; tb < nb; ++tb) {
            const float vc = owner ? sv[tb * tile_cols + local] : 0.f;
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int dd = r * ds_count + ds;
                if (dd < d) {
                    S[r] = fmaf(sa[tb * d + dd], S[r], sk[tb * d + dd] * vc);
                    o = fmaf(S[r], sq[tb * d + dd], o);
                }
            }
            for (int step = 1; step < ds_count; step <<= 1) o += __shfl_xor_sync(0xffffffffu, o, step);
            if (owner && ds == 0) {
                if (FUSED) so[tb * tile_cols + local] = o;
                else o_raw[((size_t)(first + t0 + tb) * n_heads + head) * e + col] = o;
            }
        }
        if (FUSED) {
            __syncthreads();
            gla_norm_gate_rows<T, W>(so, tile_cols, nb, (size_t)(first + t0), g, ld, norm_w, eps, n_heads, head, e, out,
                                     lane, warp, warps);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int dd = r * ds_count + ds;
        if (owner && dd < d) slot[(size_t)dd * e + col] = S[r];
    }
}

// The norm and the gate for heads whose value columns were spread over several blocks: one block per token.
template <typename T, typename W>
__global__ void __launch_bounds__(256)
gla_norm_gate_kernel(const float* __restrict__ o_raw, const T* __restrict__ g, int ld, const W* __restrict__ norm_w,
                     float eps, int n_heads, int e, T* __restrict__ out) {
    qil_wait_for_producer();
    qil_release_consumer();
    const size_t token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int head = warp; head < n_heads; head += 8)
        gla_norm_gate_rows<T, W>(o_raw + (token * n_heads + head) * e, 0, 1, token, g, ld, norm_w, eps, n_heads, head, e,
                                 out, lane, 0, 1);
}

template <typename T, typename W, bool FUSED>
static cudaError_t gla_launch(dim3 grid, int threads, size_t smem, cudaStream_t stream, const void* q, const void* k,
                              const void* v, const void* g, const void* low, int ld, const void* a2, const void* a2_bias,
                              int rank, float inv_tau, float q_scale, const void* norm_w, float eps, float* state,
                              const int* seg_start, const int* seg_len, const int* seg_row, int n_heads, int d, int e,
                              int ds_count, int tile_cols, float* o_raw, void* out) {
    cudaError_t err = cudaFuncSetAttribute(gla_scan_kernel<T, W, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    return qil_launch_chained(gla_scan_kernel<T, W, FUSED>, grid, dim3(threads), smem, stream,
                              (const T*)q, (const T*)k, (const T*)v, (const T*)g, (const T*)low, ld, (const W*)a2,
                              (const W*)a2_bias, rank, inv_tau, q_scale, (const W*)norm_w, eps, state, seg_start, seg_len,
                              seg_row, n_heads, d, e, ds_count, tile_cols, o_raw, (T*)out);
}

// o_raw: float32 [tokens, heads * e] of scratch, needed only when a head's value columns do not fit one
// block (qil_gla_scan_needs_scratch).
extern "C" int qil_gla_scan_needs_scratch(int d, int e) {
    int ds_count = 1;
    while (ds_count * GLA_R < d) ds_count <<= 1;
    return ds_count > 32 ? -1 : (e > GLA_THREADS / ds_count ? 1 : 0);
}

extern "C" int qil_gla_scan(const void* q, const void* k, const void* v, const void* g, const void* low, int ld,
                            const void* a2, const void* a2_bias, int rank, float tau, float q_scale,
                            const void* norm_w, float eps, float* state, const int* seg_start, const int* seg_len,
                            const int* seg_row, int n_segments, int n_tokens, int n_heads, int d, int e, float* o_raw,
                            void* out, int act_dtype, int weight_dtype, cudaStream_t stream) {
    if (n_segments <= 0) return 0;
    if (n_heads <= 0 || d <= 0 || e <= 0 || rank <= 0 || !(tau > 0.f) || n_segments > 65535)
        QIL_REFUSE("gla_scan: heads %d sizes %d/%d rank %d tau %g segments %d", n_heads, d, e, rank, (double)tau, n_segments);
    // a thread holds GLA_R rows of one column; ds_count threads (a power of two within a warp) share a column
    int ds_count = 1;
    while (ds_count * GLA_R < d) ds_count <<= 1;
    if (ds_count > 32) QIL_REFUSE("gla_scan: %d key channels per head are more than %d", d, 32 * GLA_R);
    const int tile_cols = e < GLA_THREADS / ds_count ? e : GLA_THREADS / ds_count;
    const int tiles = (e + tile_cols - 1) / tile_cols;
    const bool fused = tiles == 1;
    if (!fused && o_raw == nullptr) QIL_REFUSE("gla_scan: %d value columns per head need the scratch buffer", e);
    const int threads = (tile_cols * ds_count + 31) / 32 * 32;
    const size_t smem = (size_t)GLA_TB * (3 * d + 2 * tile_cols) * sizeof(float);
    dim3 grid(n_heads * tiles, n_segments);
    cudaError_t err = cudaSuccess;
#define QIL_GLA_GO(F)                                                                                            \
    QIL_DISPATCH_2(act_dtype, weight_dtype,                                                                      \
        (err = gla_launch<T, W, F>(grid, threads, smem, stream, q, k, v, g, low, ld, a2, a2_bias, rank, 1.f / tau, \
                                   q_scale, norm_w, eps, state, seg_start, seg_len, seg_row, n_heads, d, e,      \
                                   ds_count, tile_cols, o_raw, out)))
    if (fused) QIL_GLA_GO(true); else QIL_GLA_GO(false);
#undef QIL_GLA_GO
    if (err != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(err)); return (int)err; }
    if (!fused) {
        QIL_DISPATCH_2(act_dtype, weight_dtype,
            qil_launch_chained(gla_norm_gate_kernel<T, W>, dim3(n_tokens), dim3(256), 0, stream, (const float*)o_raw,
                               (const T*)g, ld, (const W*)norm_w, eps, n_heads, e, (T*)out));
    }
    QIL_CHECK_LAUNCH();
}
