// The dense operations declared in compat/full/TensorN.hpp: what CXX-GPT's model headers expect
// from the absent TensorN library.  They sit around the attention path, not on it: cuBLAS SGEMM
// for the products (pedantic fp32 unless set_tf32(true)) and plain grid-stride kernels for the
// rest.  All launches go to the legacy default stream, like the model's own kernels.
#include <cublas_v2.h>

#include <cmath>

#include "TensorN.hpp"

namespace TensorN {
namespace cuda {
namespace {

cublasHandle_t handle() {
    static cublasHandle_t h = [] {
        cublasHandle_t x;
        if (cublasCreate(&x) != CUBLAS_STATUS_SUCCESS) throw std::runtime_error("cublasCreate failed");
        cublasSetMathMode(x, CUBLAS_PEDANTIC_MATH);
        return x;
    }();
    return h;
}

unsigned blocks(size_t n) { return (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16); }

void same_size(const CudaTensor<float>& a, const CudaTensor<float>& b, const char* what) {
    if (a.size() != b.size()) throw std::runtime_error(std::string(what) + ": size mismatch");
}

__global__ void transpose_kernel(const float* __restrict__ A, float* __restrict__ At, size_t m, size_t n) {
    __shared__ float tile[32][33];
    const size_t bx = (size_t)blockIdx.x * 32, by = (size_t)blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const size_t r = by + j, c = bx + threadIdx.x;
        if (r < m && c < n) tile[j][threadIdx.x] = A[r * n + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const size_t r = bx + j, c = by + threadIdx.x;  // row of At = column of A
        if (r < n && c < m) At[r * m + c] = tile[threadIdx.x][j];
    }
}

template <int OP>
__global__ void binary_kernel(const float* A, const float* B, float* C, size_t n, float s) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        C[i] = OP == 0 ? A[i] + B[i] : OP == 1 ? A[i] * B[i] : A[i] * s;
}

__global__ void column_sum_kernel(const float* __restrict__ A, float* __restrict__ out, size_t m, size_t n) {
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n) return;
    float acc = 0.f;
    for (size_t r = 0; r < m; r++) acc += A[r * n + c];
    out[c] = acc;
}

__global__ void row_sum_kernel(const float* __restrict__ A, float* __restrict__ out, size_t m, size_t n) {
    const size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= m) return;
    float acc = 0.f;
    for (size_t c = 0; c < n; c++) acc += A[r * n + c];
    out[r] = acc;
}

// one warp per row
__global__ void softmax_rows_kernel(const float* __restrict__ A, float* __restrict__ out, size_t rows, size_t n) {
    const size_t r = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    const int lane = threadIdx.x % 32;
    if (r >= rows) return;
    const float* a = A + r * n;
    float mx = -INFINITY;
    for (size_t c = lane; c < n; c += 32) mx = fmaxf(mx, a[c]);
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (size_t c = lane; c < n; c += 32) sum += expf(a[c] - mx);
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (size_t c = lane; c < n; c += 32) out[r * n + c] = expf(a[c] - mx) * inv;
}

__global__ void gelu_tanh_kernel(const float* A, float* out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = A[i];
        out[i] = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    }
}

void launched() { CHECK_CUDA_ERROR(cudaGetLastError()); }

}  // namespace

void set_tf32(bool on) { cublasSetMathMode(handle(), on ? CUBLAS_TF32_TENSOR_OP_MATH : CUBLAS_PEDANTIC_MATH); }

void matmul(const CudaTensor<float>& A, const CudaTensor<float>& B, CudaTensor<float>& C) {
    const auto &sa = A.shape(), &sb = B.shape();
    if (sa.size() != 2 || sb.size() != 2 || sa[1] != sb[0] || C.size() != sa[0] * sb[1])
        throw std::runtime_error("matmul: shape mismatch");
    const int m = (int)sa[0], k = (int)sa[1], n = (int)sb[1];
    const float one = 1.0f, zero = 0.0f;
    // row-major C = A B  <=>  column-major C^T = B^T A^T
    if (cublasSgemm(handle(), CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, &one, B.device_ptr(), n, A.device_ptr(), k, &zero,
                    C.device_ptr(), n) != CUBLAS_STATUS_SUCCESS)
        throw std::runtime_error("cublasSgemm failed");
}

void transpose(const CudaTensor<float>& A, CudaTensor<float>& At) {
    const auto& s = A.shape();
    if (s.size() != 2 || At.size() != A.size()) throw std::runtime_error("transpose: shape mismatch");
    const dim3 grid((unsigned)((s[1] + 31) / 32), (unsigned)((s[0] + 31) / 32));
    transpose_kernel<<<grid, dim3(32, 8)>>>(A.device_ptr(), At.device_ptr(), s[0], s[1]);
    launched();
}

void add(const CudaTensor<float>& A, const CudaTensor<float>& B, CudaTensor<float>& C) {
    same_size(A, B, "add");
    same_size(A, C, "add");
    if (!A.size()) return;
    binary_kernel<0><<<blocks(A.size()), 256>>>(A.device_ptr(), B.device_ptr(), C.device_ptr(), A.size(), 0.f);
    launched();
}

void multiply(const CudaTensor<float>& A, const CudaTensor<float>& B, CudaTensor<float>& C) {
    same_size(A, B, "multiply");
    same_size(A, C, "multiply");
    if (!A.size()) return;
    binary_kernel<1><<<blocks(A.size()), 256>>>(A.device_ptr(), B.device_ptr(), C.device_ptr(), A.size(), 0.f);
    launched();
}

void multiply_scalar(const CudaTensor<float>& A, float s, CudaTensor<float>& C) {
    same_size(A, C, "multiply_scalar");
    if (!A.size()) return;
    binary_kernel<2><<<blocks(A.size()), 256>>>(A.device_ptr(), A.device_ptr(), C.device_ptr(), A.size(), s);
    launched();
}

CudaTensor<float> sum_axis(const CudaTensor<float>& A, int axis) {
    const auto& s = A.shape();
    if (s.size() != 2 || (axis != 0 && axis != 1)) throw std::runtime_error("sum_axis: only 2-D, axis 0 or 1");
    CudaTensor<float> out({axis == 0 ? s[1] : s[0]});
    if (axis == 0) column_sum_kernel<<<(unsigned)((s[1] + 127) / 128), 128>>>(A.device_ptr(), out.device_ptr(), s[0], s[1]);
    else row_sum_kernel<<<(unsigned)((s[0] + 127) / 128), 128>>>(A.device_ptr(), out.device_ptr(), s[0], s[1]);
    launched();
    return out;
}

void softmax(const CudaTensor<float>& A, CudaTensor<float>& out, int axis) {
    const auto& s = A.shape();
    if (s.empty() || (axis != -1 && axis != (int)s.size() - 1)) throw std::runtime_error("softmax: last axis only");
    same_size(A, out, "softmax");
    const size_t n = s.back(), rows = A.size() / n;
    softmax_rows_kernel<<<(unsigned)((rows + 7) / 8), 256>>>(A.device_ptr(), out.device_ptr(), rows, n);
    launched();
}

void gelu(const CudaTensor<float>& A, CudaTensor<float>& out) {
    same_size(A, out, "gelu");
    if (!A.size()) return;
    gelu_tanh_kernel<<<blocks(A.size()), 256>>>(A.device_ptr(), out.device_ptr(), A.size());
    launched();
}

}  // namespace cuda
}  // namespace TensorN
