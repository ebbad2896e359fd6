// A short causal convolution over time on every channel of a stacked projection, as the tail of a
// q/k/v projection: for the token at position t of its sequence and channel c,
//
//   y_t[c] = sum_{j < taps} w[c][j] * u_(t - taps + 1 + j)[c],      u = 0 before the sequence's start.
//
// The convolved queries go to their buffer, the convolved keys and values into the request's pages
// (a page holds its key rows [kv_head][slot][head_dim] followed by its value rows [kv_head][slot][v_dim]).
// The u of earlier positions come from the step's own rows when the same request brought them in this
// step (a request's tokens are consecutive rows at consecutive positions), else from the request's
// state slot, which holds the last taps - 1 rows of u that earlier steps saw: float32
// [slot][taps - 1][channels], the newest last, zeroed at admission.  The sum runs over j in ascending
// order with float32 FMA and is rounded once to the activation type, so a token's result does not
// depend on how its sequence was cut into steps.  The weights come as [taps][channels] (the checkpoint's
// [channels][taps] transposed once after loading), so that a tap's weights of neighbouring channels lie side by side.
//
// Two kernels: the convolution (one block per token), which also moves the state of a request that
// brought exactly one token (it is the only reader of that slot), and the state update for requests
// that brought more (one block per segment and slab of channels, after the convolution has read the
// old state).  With n_kv_heads == 0 only queries exist (a layer that reads another layer's pages).
#include "common.cuh"

#define CONV_MAX_TAPS 16

template <typename T, typename W>
__global__ void __launch_bounds__(256)
short_conv_store_kernel(const T* __restrict__ u, const W* __restrict__ taps_w, float* __restrict__ state,
                        T* __restrict__ q_out, T* __restrict__ kv_cache, const int* __restrict__ positions,
                        const int* __restrict__ token_row, const int* __restrict__ block_table, int table_stride,
                        int n_tokens, int taps, int n_q_heads, int n_kv_heads, int head_dim, int v_dim, int page_size,
                        int num_pages) {
    qil_wait_for_producer();
    qil_release_consumer();
    const int token = blockIdx.x;
    const int pos = positions[token], row = token_row[token];
    const int q_width = n_q_heads * head_dim, k_width = n_kv_heads * head_dim, v_width = n_kv_heads * v_dim;
    const int channels = q_width + k_width + v_width;
    // how many earlier positions this step itself brought (at most taps - 1 matter)
    int history = 0;
    while (history < taps - 1 && token - history - 1 >= 0 && token_row[token - history - 1] == row
           && positions[token - history - 1] == pos - history - 1)
        ++history;
    const bool alone = history == 0 && (token + 1 >= n_tokens || token_row[token + 1] != row);
    const float* slot = state + (size_t)row * (taps - 1) * channels;
    T* k_page = nullptr;
    T* v_page = nullptr;
    int slot_in_page = 0;
    if (n_kv_heads > 0) {
        const int index = pos / page_size;
        const int page = (pos >= 0 && index < table_stride) ? block_table[(size_t)row * table_stride + index] : -1;
        if (page >= 0 && page < num_pages) {      // never write outside the pool
            k_page = kv_cache + (size_t)page * n_kv_heads * page_size * (head_dim + v_dim);
            v_page = k_page + (size_t)n_kv_heads * page_size * head_dim;
            slot_in_page = pos % page_size;
        }
    }
    for (int c = threadIdx.x; c < channels; c += 256) {
        float window[CONV_MAX_TAPS];       // u at positions pos - taps + 1 + j
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            float value = 0.f;
            if (j < taps) {
                const int back = taps - 1 - j;             // how far behind this token
                if (back <= history) value = to_f32<T>(u[(size_t)(token - back) * channels + c]);
                else if (pos - back >= 0) value = slot[(size_t)(taps - 1 - (back - history)) * channels + c];
            }
            window[j] = value;
        }
        float y = 0.f;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j < taps) y = fmaf(to_f32<W>(taps_w[(size_t)j * channels + c]), window[j], y);
        const T result = from_f32<T>(y);
        if (c < q_width) {
            q_out[(size_t)token * q_width + c] = result;
        } else if (c < q_width + k_width) {
            const int i = c - q_width;
            if (k_page != nullptr) k_page[((size_t)(i / head_dim) * page_size + slot_in_page) * head_dim + i % head_dim] = result;
        } else {
            const int i = c - q_width - k_width;
            if (v_page != nullptr) v_page[((size_t)(i / v_dim) * page_size + slot_in_page) * v_dim + i % v_dim] = result;
        }
        if (alone) {       // the request's only token of the step: its state moves on by one row, here
            float* mine = state + (size_t)row * (taps - 1) * channels;
#pragma unroll
            for (int j = 1; j < CONV_MAX_TAPS; ++j)
                if (j < taps) mine[(size_t)(j - 1) * channels + c] = (pos - (taps - 1 - j) >= 0) ? window[j] : 0.f;
        }
    }
}


// The same for bfloat16 rows and weights whose sizes allow 16-byte moves (channels, head sizes multiples of 8, at
// most 8 taps): a thread owns 8 consecutive channels, which never straddle a head, so a token's row is read in
// 16-byte pieces and every key and value row of a page is written in them.  The arithmetic is the scalar kernel's:
// float32 FMA over j in ascending order, one rounding.
#define CONV_VEC_TAPS 8
__device__ __forceinline__ void conv_unpack8(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(pairs[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
}

__global__ void __launch_bounds__(128)
short_conv_store_vec8_kernel(const bf16* __restrict__ u, const bf16* __restrict__ taps_w, float* __restrict__ state,
                             bf16* __restrict__ q_out, bf16* __restrict__ kv_cache, const int* __restrict__ positions,
                             const int* __restrict__ token_row, const int* __restrict__ block_table, int table_stride,
                             int n_tokens, int taps, int n_q_heads, int n_kv_heads, int head_dim, int v_dim, int page_size,
                             int num_pages) {
    qil_wait_for_producer();
    qil_release_consumer();
    const int token = blockIdx.x;
    const int pos = positions[token], row = token_row[token];
    const int q_width = n_q_heads * head_dim, k_width = n_kv_heads * head_dim, v_width = n_kv_heads * v_dim;
    const int channels = q_width + k_width + v_width;
    const int c = (blockIdx.y * 128 + threadIdx.x) * 8;
    if (c >= channels) return;
    int history = 0;
    while (history < taps - 1 && token - history - 1 >= 0 && token_row[token - history - 1] == row
           && positions[token - history - 1] == pos - history - 1)
        ++history;
    const bool alone = history == 0 && (token + 1 >= n_tokens || token_row[token + 1] != row);
    float* slot = state + (size_t)row * (taps - 1) * channels;
    float y[8];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) y[ch] = 0.f;
    float newest[CONV_VEC_TAPS][8];          // the rows of u behind this token and its own: what an alone token's state becomes
#pragma unroll
    for (int j = 0; j < CONV_VEC_TAPS; ++j) {
        float value[8];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) value[ch] = 0.f;
        if (j < taps) {
            const int back = taps - 1 - j;
            if (back <= history) {
                conv_unpack8(*reinterpret_cast<const uint4*>(u + (size_t)(token - back) * channels + c), value);
            } else if (pos - back >= 0) {
                const float4* src = reinterpret_cast<const float4*>(slot + (size_t)(taps - 1 - (back - history)) * channels + c);
                const float4 a = src[0], b = src[1];
                value[0] = a.x; value[1] = a.y; value[2] = a.z; value[3] = a.w;
                value[4] = b.x; value[5] = b.y; value[6] = b.z; value[7] = b.w;
            }
            float w[8];        // tap j of this thread's 8 channels: 16 bytes of the [taps][channels] weights
            conv_unpack8(*reinterpret_cast<const uint4*>(taps_w + (size_t)j * channels + c), w);
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) y[ch] = fmaf(w[ch], value[ch], y[ch]);
        }
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) newest[j][ch] = value[ch];
    }
    uint4 packed;
    __nv_bfloat162* halves = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) halves[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
    if (c < q_width) {
        *reinterpret_cast<uint4*>(q_out + (size_t)token * q_width + c) = packed;
    } else if (n_kv_heads > 0) {
        const int index = pos / page_size;
        const int page = (pos >= 0 && index < table_stride) ? block_table[(size_t)row * table_stride + index] : -1;
        if (page >= 0 && page < num_pages) {      // never write outside the pool
            bf16* k_page = kv_cache + (size_t)page * n_kv_heads * page_size * (head_dim + v_dim);
            const int slot_in_page = pos % page_size;
            if (c < q_width + k_width) {
                const int i = c - q_width;
                *reinterpret_cast<uint4*>(k_page + ((size_t)(i / head_dim) * page_size + slot_in_page) * head_dim + i % head_dim) = packed;
            } else {
                const int i = c - q_width - k_width;
                bf16* v_page = k_page + (size_t)n_kv_heads * page_size * head_dim;
                *reinterpret_cast<uint4*>(v_page + ((size_t)(i / v_dim) * page_size + slot_in_page) * v_dim + i % v_dim) = packed;
            }
        }
    }
    if (alone) {
#pragma unroll
        for (int j = 1; j < CONV_VEC_TAPS; ++j)
            if (j < taps) {
                const bool real = pos - (taps - 1 - j) >= 0;
                float4* dst = reinterpret_cast<float4*>(slot + (size_t)(j - 1) * channels + c);
                dst[0] = real ? make_float4(newest[j][0], newest[j][1], newest[j][2], newest[j][3]) : make_float4(0.f, 0.f, 0.f, 0.f);
                dst[1] = real ? make_float4(newest[j][4], newest[j][5], newest[j][6], newest[j][7]) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
    }
}

// The state after a segment of more than one token: the last taps - 1 rows of u that the request has seen.
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const T* __restrict__ u, float* __restrict__ state, const int* __restrict__ seg_row,
                        const int* __restrict__ seg_start, const int* __restrict__ seg_len, int taps, int channels) {
    qil_wait_for_producer();
    qil_release_consumer();
    const int segment = blockIdx.x;
    const int len = seg_len[segment];
    if (len <= 1) return;                 // the convolution kernel moved that state itself
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= channels) return;
    const int first = seg_start[segment];
    float* slot = state + (size_t)seg_row[segment] * (taps - 1) * channels;
    float rows[CONV_MAX_TAPS];
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {
        const int at = len - (taps - 1) + i;          // index into the segment; negative: before it
        rows[i] = 0.f;
        if (i < taps - 1)
            rows[i] = at >= 0 ? to_f32<T>(u[(size_t)(first + at) * channels + c]) : slot[(size_t)(len + i) * channels + c];
    }
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i)
        if (i < taps - 1) slot[(size_t)i * channels + c] = rows[i];
}

extern "C" int qil_short_conv_store(const void* u, const void* taps_w, float* state, void* q_out, void* kv_cache,
                                    const int* positions, const int* token_row, const int* block_table,
                                    int table_stride, int n_tokens, int taps, int n_q_heads, int n_kv_heads,
                                    int head_dim, int v_dim, int page_size, int num_pages, int act_dtype,
                                    int weight_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS) QIL_REFUSE("short_conv: %d taps (1 to %d)", taps, CONV_MAX_TAPS);
    if (n_q_heads <= 0 || n_kv_heads < 0 || head_dim <= 0 || v_dim <= 0 || page_size <= 0)
        QIL_REFUSE("short_conv: heads %d/%d sizes %d/%d page %d", n_q_heads, n_kv_heads, head_dim, v_dim, page_size);
    const int channels = n_q_heads * head_dim + n_kv_heads * (head_dim + v_dim);
    if (act_dtype == QIL_BF16 && weight_dtype == QIL_BF16 && taps <= CONV_VEC_TAPS && head_dim % 8 == 0 && v_dim % 8 == 0
        && (((uintptr_t)u | (uintptr_t)taps_w | (uintptr_t)state | (uintptr_t)q_out | (uintptr_t)kv_cache) & 15) == 0) {
        qil_launch_chained(short_conv_store_vec8_kernel, dim3(n_tokens, (channels / 8 + 127) / 128), dim3(128), 0, stream,
                           (const bf16*)u, (const bf16*)taps_w, state, (bf16*)q_out, (bf16*)kv_cache, positions, token_row,
                           block_table, table_stride, n_tokens, taps, n_q_heads, n_kv_heads, head_dim, v_dim, page_size,
                           num_pages);
        QIL_CHECK_LAUNCH();
    }
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        qil_launch_chained(short_conv_store_kernel<T, W>, dim3(n_tokens), dim3(256), 0, stream, (const T*)u,
                           (const W*)taps_w, state, (T*)q_out, (T*)kv_cache, positions, token_row, block_table,
                           table_stride, n_tokens, taps, n_q_heads, n_kv_heads, head_dim, v_dim, page_size, num_pages));
    QIL_CHECK_LAUNCH();
}

extern "C" int qil_short_conv_state(const void* u, float* state, const int* seg_row, const int* seg_start,
                                    const int* seg_len, int n_segments, int taps, int channels, int act_dtype,
                                    cudaStream_t stream) {
    if (n_segments <= 0 || taps <= 1) return 0;
    if (taps > CONV_MAX_TAPS || channels <= 0) QIL_REFUSE("short_conv_state: %d taps, %d channels", taps, channels);
    dim3 grid(n_segments, (channels + 255) / 256);
    QIL_DISPATCH_1(act_dtype,
        qil_launch_chained(short_conv_state_kernel<T>, grid, dim3(256), 0, stream, (const T*)u, state, seg_row,
                           seg_start, seg_len, taps, channels));
    QIL_CHECK_LAUNCH();
}
