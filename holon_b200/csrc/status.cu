// The host's view of the kernels' bounded waits. Every wait inside a kernel (on an mbarrier in the tcgen05 kernels, on
// the grid barrier and the hand-over flags of the chained products) gives up after a fixed number of polls and records
// where (tcgen05.cuh). Reading those words needs a copy from the device; a serving
// loop cannot afford one per step. So one word of page-locked host memory, mapped into the device's address space, is
// handed to every kernel file as its mirror: a wait that gives up writes its code there as well, and the host reads
// that word, in its own memory, whenever a step's completion event has fired.
#include "tcgen05.cuh"

extern "C" int hb_attention_tcgen05_status_mirror(unsigned int* word);
extern "C" int hb_gemm_tcgen05_status_mirror(unsigned int* word);
extern "C" int hb_gemm_tcgen05_pair_status_mirror(unsigned int* word);
extern "C" int hb_gemm_chain_status_mirror(unsigned int* word);
extern "C" int hb_gemm_tickets_status_mirror(unsigned int* word);
extern "C" int hb_gemm_mid_status_mirror(unsigned int* word);
HB_DEFINE_STATUS_MIRROR(hb_status_selftest_mirror)

static unsigned int* g_word_host = nullptr;
static unsigned int* g_word_device = nullptr;

// The host address of the status word (made, and handed to the kernel files of the current device, at the first
// call). 0 there: every wait so far ended; else (place << 28) | (block + 1) of a wait that gave up. The host may write
// 0 to it to start afresh.
extern "C" int hb_status_word(unsigned int** host) {
    if (g_word_host == nullptr) {
        unsigned int* word = nullptr;
        HB_CUDA(cudaHostAlloc((void**)&word, sizeof(unsigned int), cudaHostAllocMapped | cudaHostAllocPortable));
        *word = 0;
        unsigned int* device = nullptr;
        HB_CUDA(cudaHostGetDevicePointer((void**)&device, word, 0));
        if (hb_attention_tcgen05_status_mirror(device) || hb_gemm_tcgen05_status_mirror(device) ||
            hb_gemm_tcgen05_pair_status_mirror(device) || hb_gemm_chain_status_mirror(device) ||
            hb_gemm_tickets_status_mirror(device) || hb_gemm_mid_status_mirror(device) ||
            hb_status_selftest_mirror(device))
            return HB_ERR_CUDA;
        g_word_host = word;
        g_word_device = device;
    }
    *host = g_word_host;
    return 0;
}

// The same word's address as the device sees it, for kernel files outside this library (a part's own): they hand it
// to their HB_DEFINE_STATUS_MIRROR function, and their waits report like every other.
extern "C" int hb_status_word_device(unsigned int** device) {
    unsigned int* host = nullptr;
    if (int code = hb_status_word(&host)) return code;
    *device = g_word_device;
    return 0;
}

// A wait that runs out, for tests of what the host does then: one warp polls `polls` times an mbarrier at which
// nobody ever arrives, gives up as the kernels' waits do (place 15) and returns. It takes microseconds and leaves
// the device as it was.
__global__ void status_selftest_kernel(unsigned polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_addr(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        mbar_wait_limit(smem_addr(&bar), 0, 15u, polls);
    }
}

extern "C" int hb_status_selftest(int polls, hb_stream stream) {
    if (polls < 1 || polls > (1 << 20)) HB_REFUSE("status_selftest: 1 to 2^20 polls, not %d", polls);
    status_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned)polls);
    HB_LAUNCH_CHECK("status_selftest");
    return 0;
}
