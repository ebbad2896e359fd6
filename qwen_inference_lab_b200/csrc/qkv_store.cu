// The tail of a q/k/v projection for attention without rotation: queries are copied to their buffer,
// multiplied by a temperature that grows with the logarithm of the position where one is set,
//
//   q'_p = q_p * (1 + coef * ln(floor((p + 1) / every) + 1)),
//
// and keys and values go into the request's pages.  Keys and values may differ in size: a page holds
// its key rows [kv_head][slot][head_dim] followed by its value rows [kv_head][slot][v_dim].  The
// temperature is computed in float32 from the integer position; the product is rounded once.
// With n_kv_heads == 0 only queries are processed (a layer that reads another layer's pages).
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
qkv_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ kv_cache,
                 const int* __restrict__ positions, const int* __restrict__ token_row,
                 const int* __restrict__ block_table, int table_stride, int n_q_heads, int n_kv_heads,
                 int head_dim, int v_dim, int page_size, int num_pages, float temp_coef, int temp_every) {
    qil_wait_for_producer();
    qil_release_consumer();
    const int token = blockIdx.x;
    const int pos = positions[token];
    const int q_width = n_q_heads * head_dim, k_width = n_kv_heads * head_dim, v_width = n_kv_heads * v_dim;
    const T* src = qkv + (size_t)token * (q_width + k_width + v_width);
    float temperature = 1.f;
    if (temp_coef != 0.f && temp_every > 0) temperature = 1.f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.f);
    T* q_dst = q_out + (size_t)token * q_width;
    for (int i = threadIdx.x; i < q_width; i += 256) q_dst[i] = from_f32<T>(to_f32<T>(src[i]) * temperature);
    if (n_kv_heads == 0) return;
    const int index = pos / page_size;
    const int page = (pos >= 0 && index < table_stride) ? block_table[(size_t)token_row[token] * table_stride + index] : -1;
    if (page < 0 || page >= num_pages) return;      // never write outside the pool
    const int slot = pos % page_size;
    T* page_base = kv_cache + (size_t)page * n_kv_heads * page_size * (head_dim + v_dim);
    for (int i = threadIdx.x; i < k_width; i += 256) {
        const int head = i / head_dim, d = i % head_dim;
        page_base[((size_t)head * page_size + slot) * head_dim + d] = src[q_width + i];
    }
    T* v_base = page_base + (size_t)n_kv_heads * page_size * head_dim;
    for (int i = threadIdx.x; i < v_width; i += 256) {
        const int head = i / v_dim, d = i % v_dim;
        v_base[((size_t)head * page_size + slot) * v_dim + d] = src[q_width + k_width + i];
    }
}

extern "C" int qil_qkv_store(const void* qkv, void* q_out, void* kv_cache, const int* positions, const int* token_row,
                             const int* block_table, int table_stride, int n_tokens, int n_q_heads, int n_kv_heads,
                             int head_dim, int v_dim, int page_size, int num_pages, float temp_coef, int temp_every,
                             int act_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_q_heads <= 0 || n_kv_heads < 0 || head_dim <= 0 || v_dim <= 0 || page_size <= 0)
        QIL_REFUSE("qkv_store: heads %d/%d sizes %d/%d page %d", n_q_heads, n_kv_heads, head_dim, v_dim, page_size);
    QIL_DISPATCH_1(act_dtype,
        qil_launch_chained(qkv_store_kernel<T>, dim3(n_tokens), dim3(256), 0, stream,
                           (const T*)qkv, (T*)q_out, (T*)kv_cache, positions, token_row, block_table, table_stride,
                           n_q_heads, n_kv_heads, head_dim, v_dim, page_size, num_pages, temp_coef, temp_every));
    QIL_CHECK_LAUNCH();
}
