// Host-side support shared by every entry point of libbongard_b200: error text, device
// check, the TMA descriptor encoder (resolved from the driver at run time, so the library
// links against the CUDA runtime only) and the status word that bounded waits report to.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace {

thread_local char g_error[512] = "";

// One status word per device, living in the module's own global memory: nothing is allocated.
__device__ int32_t g_status_word = 0;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

void bg_set_error(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
}

int bg_make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                       CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) {
        bg_set_error("cuTensorMapEncodeTiled is not available from this driver");
        return BG_ERR_DRIVER;
    }
    cuuint64_t d[5];
    cuuint64_t s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
    CUresult r = fn(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        bg_set_error("cuTensorMapEncodeTiled failed with code %d (rank %d, dims %llu x %llu, stride %llu, box %u x %u)",
                     (int)r, rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0),
                     (unsigned long long)(rank > 1 ? strides_bytes[0] : 0), box[0], rank > 1 ? box[1] : 0);
        return BG_ERR_DRIVER;
    }
    return BG_OK;
}

int bg_device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kBgMaxDevices) return 0;
    return dev;
}

// Every cache below is a table indexed by the current device: a process that drives several GPUs
// gets each device's own SM count, status word and kernel attributes.
int bg_num_sms() {
    static int sms[kBgMaxDevices] = {};
    const int dev = bg_device_slot();
    if (!sms[dev]) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms[dev] = n > 0 ? n : 148;
    }
    return sms[dev];
}

int32_t* bg_status_word() {
    static int32_t* ptr[kBgMaxDevices] = {};
    const int dev = bg_device_slot();
    if (!ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {     // the symbol's address on the CURRENT device
            bg_set_error("cudaGetSymbolAddress(status word) failed");
            return nullptr;
        }
        ptr[dev] = static_cast<int32_t*>(p);
    }
    return ptr[dev];
}

// Self-test of the bounded wait: one CTA waits on a barrier phase that nothing completes, with the
// caller's budget instead of the kernels' 4 s.  When the budget runs out the wait reports site 901
// to the status word and returns false, as it does inside the GEMM and attention kernels; every
// thread then takes the normal way out.  Nothing traps, faults or spins past the budget.
__global__ void bounded_wait_selftest_kernel(int32_t* status, uint64_t budget_ns, int32_t* finished) {
    using namespace bg;
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    Abort ab{&abort_flag, status};
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(&bar, 0, ab, 901, budget_ns);     // nobody arrives: runs out
    __syncthreads();
    // the other threads see the CTA-wide abort flag, as the kernels' later waits do
    if (threadIdx.x == 1 && finished) *finished = ab.raised() ? 1 : 0;
    (void)ok;
}

static int g_programmatic_launch = 0;
int bg_programmatic_launch() { return g_programmatic_launch; }

extern "C" {

// 1: launch the kernels of the serving chain (GEMMs, attention, norms, head) with programmatic stream
// serialization, so that a kernel's prologue overlaps the tail of its predecessor; 0 (default): plain launches.
void bg_set_programmatic_launch(int enable) { g_programmatic_launch = enable ? 1 : 0; }

const char* bg_last_error_string() { return g_error; }

int bg_version() { return 1; }

// 0 when the current device is an sm_100 part the kernels were compiled for.
int bg_device_check() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        bg_set_error("no CUDA device: %s", cudaGetErrorString(e));
        return BG_ERR_ARCH;
    }
    int major = 0, minor = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (major != 10) {
        bg_set_error("libbongard_b200 is built for sm_100a only; device %d is sm_%d%d", dev, major, minor);
        return BG_ERR_ARCH;
    }
    if (!encode_tiled()) {
        bg_set_error("cuTensorMapEncodeTiled is not available from this driver");
        return BG_ERR_DRIVER;
    }
    return BG_OK;
}

// Reads and clears the status word after synchronising `stream`.  0 = every bounded wait completed;
// otherwise the code of the first wait that ran out (1xx GEMM, 2xx attention, 3xx FP8 GEMM).
int bg_read_status(void* stream) {
    int32_t* word = bg_status_word();
    if (!word) return BG_ERR_DRIVER;
    int32_t host = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&host, word, sizeof(host), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        bg_set_error("bg_read_status: %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    if (host != 0) {
        cudaMemsetAsync(word, 0, sizeof(host), s);
        cudaStreamSynchronize(s);
        bg_set_error("a bounded device wait ran out (site %d)", host);
    }
    return host;
}

// Launches the bounded-wait self-test (see bounded_wait_selftest_kernel) with a budget of
// `budget_us` microseconds (1 .. 100000).  `finished` (device int32, may be NULL) is set to 1 by
// the kernel after the wait gave up.  bg_read_status(stream) afterwards returns 901.
int bg_selftest_bounded_wait(int64_t budget_us, int32_t* finished, void* stream) {
    if (budget_us < 1 || budget_us > 100000) {
        bg_set_error("bg_selftest_bounded_wait: budget must be 1..100000 microseconds");
        return BG_ERR_SHAPE;
    }
    int32_t* word = bg_status_word();
    if (!word) return BG_ERR_DRIVER;
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(word, (uint64_t)budget_us * 1000ull, finished);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        bg_set_error("bg_selftest_bounded_wait: %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

}  // extern "C"
