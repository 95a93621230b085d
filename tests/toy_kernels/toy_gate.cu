// A toy part's own CUDA file, for the test of the kernel table's extension seam: it is compiled into a library of its
// own, beside the engine's, and called through the table. out = x * sigmoid(scale * x), column by column, in 32-bit.
// Its second function is a wait that runs out (a barrier nobody arrives at), to show that a bounded wait in a part's
// own kernel reaches the engine's status word.
#include "tcgen05.cuh"

template <typename T>
__global__ void toy_gate_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ scale, int rows, int dim) {
    const size_t n = (size_t)rows * dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = to_f32(x[i]);
        out[i] = from_f32<T>(v / (1.f + __expf(-scale[i % dim] * v)));
    }
}

extern "C" int toy_gate(void* out, const void* x, int dtype, const float* scale, int rows, int dim, hb_stream stream) {
    if (rows == 0) return 0;
    if (rows < 0 || dim < 1) HB_REFUSE("toy_gate: %d rows of %d columns", rows, dim);
    if (dtype != HB_F32 && dtype != HB_BF16) HB_REFUSE("toy_gate: dtype %d", dtype);
    const int blocks = (int)(((size_t)rows * dim + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32) toy_gate_kernel<float><<<blocks, 256, 0, s>>>((float*)out, (const float*)x, scale, rows, dim);
    else toy_gate_kernel<bf16><<<blocks, 256, 0, s>>>((bf16*)out, (const bf16*)x, scale, rows, dim);
    HB_LAUNCH_CHECK("toy_gate");
    return 0;
}

HB_DEFINE_STATUS_MIRROR(toy_status_mirror)

__global__ void toy_wait_kernel(unsigned polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_addr(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        mbar_wait_limit(smem_addr(&bar), 0, 14u, polls);       // gives up after `polls` polls: place 14
    }
}

extern "C" int toy_wait_that_runs_out(int polls, hb_stream stream) {
    if (polls < 1 || polls > 4096) HB_REFUSE("toy_wait_that_runs_out: 1 to 4096 polls, not %d", polls);
    toy_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned)polls);
    HB_LAUNCH_CHECK("toy_wait_that_runs_out");
    return 0;
}
