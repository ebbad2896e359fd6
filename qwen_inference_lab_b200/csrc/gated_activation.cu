// out = act(gate) * f(up) over rows that hold the gate columns followed by the up columns (or, with
// `pairs8`, groups of 8 gate columns followed by their 8 up columns).  The kinds:
//
//   0  silu:           g sigmoid(g) * u
//   1  gelu (tanh):    0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * u
//   2  clamped swish:  g' = min(g, limit), u' = clamp(u, -limit, limit);  g' sigmoid(alpha g') * (u' + 1)
//
// The arithmetic is float32; the result is rounded once to the output type.
#include "common.cuh"

#define QIL_ACT_SILU 0
#define QIL_ACT_GELU_TANH 1
#define QIL_ACT_CLAMPED_SWISH 2

__device__ __forceinline__ float gated_value(int kind, float g, float u, float limit, float alpha) {
    if (kind == QIL_ACT_SILU) return g / (1.f + expf(-g)) * u;
    if (kind == QIL_ACT_GELU_TANH) {
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.f + tanhf(inner)) * u;
    }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, size_t total, int width, int pairs8,
                        int kind, float limit, float alpha) {
    qil_wait_for_producer();
    qil_release_consumer();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const size_t row = i / width;
        const int col = (int)(i % width);
        const T* src = gate_up + row * 2 * width;
        const int g_at = pairs8 ? (col / 8) * 16 + (col % 8) : col;
        const int u_at = pairs8 ? g_at + 8 : col + width;
        out[i] = from_f32<T>(gated_value(kind, to_f32<T>(src[g_at]), to_f32<T>(src[u_at]), limit, alpha));
    }
}

extern "C" int qil_gated_activation(const void* gate_up, void* out, int n_rows, int width, int act_dtype, int pairs8,
                                    int kind, float limit, float alpha, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || kind < 0 || kind > 2) QIL_REFUSE("gated_activation: width %d kind %d", width, kind);
    if (pairs8 && width % 8) QIL_REFUSE("gated_activation: the paired layout needs a width that is a multiple of 8");
    const size_t total = (size_t)n_rows * width;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    QIL_DISPATCH_1(act_dtype,
        qil_launch_chained(gated_activation_kernel<T>, dim3(blocks), dim3(256), 0, stream,
                           (const T*)gate_up, (T*)out, total, width, pairs8, kind, limit, alpha));
    QIL_CHECK_LAUNCH();
}

// ------------------------------------------------------------------ activations without a gate
//   0 silu   1 gelu (tanh)   3 squared relu: max(z, 0)^2
// out = act(z), or with `table`: out[r][c] = act(z[r][c]) * table[ids[r]][first_col + c], a slice of the row
// that the token's id names in a table of per-token vectors.  float32 arithmetic, one rounding.
#define QIL_ACT_RELU2 3

__device__ __forceinline__ float plain_activation(int kind, float z) {
    if (kind == QIL_ACT_SILU) return z / (1.f + expf(-z));
    if (kind == QIL_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    const float r = fmaxf(z, 0.f);
    return r * r;
}

template <typename T, typename W>
__global__ void __launch_bounds__(256)
activation_kernel(const T* __restrict__ z, T* __restrict__ out, size_t total, int width, int kind,
                  const W* __restrict__ table, const int* __restrict__ ids, int table_width, int first_col, int table_rows) {
    qil_wait_for_producer();
    qil_release_consumer();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        float v = plain_activation(kind, to_f32<T>(z[i]));
        if (table != nullptr) {
            int id = ids[i / width];
            id = id < 0 ? 0 : (id >= table_rows ? table_rows - 1 : id);
            v *= to_f32<W>(table[(size_t)id * table_width + first_col + (int)(i % width)]);
        }
        out[i] = from_f32<T>(v);
    }
}

extern "C" int qil_activation(const void* z, void* out, int n_rows, int width, int act_dtype, int kind,
                              const void* table, int table_dtype, const int* ids, int table_width, int first_col,
                              int table_rows, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || (kind != QIL_ACT_SILU && kind != QIL_ACT_GELU_TANH && kind != QIL_ACT_RELU2))
        QIL_REFUSE("activation: width %d kind %d", width, kind);
    if (table != nullptr && (ids == nullptr || first_col < 0 || first_col + width > table_width || table_rows < 1))
        QIL_REFUSE("activation: columns %d..%d of a table %d wide", first_col, first_col + width, table_width);
    const size_t total = (size_t)n_rows * width;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    QIL_DISPATCH_2(act_dtype, table != nullptr ? table_dtype : act_dtype,
        qil_launch_chained(activation_kernel<T, W>, dim3(blocks), dim3(256), 0, stream, (const T*)z, (T*)out, total,
                           width, kind, (const W*)table, ids, table_width, first_col, table_rows));
    QIL_CHECK_LAUNCH();
}
