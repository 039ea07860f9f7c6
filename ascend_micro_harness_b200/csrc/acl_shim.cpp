// The sixteen ACL runtime calls the reference's device harnesses make
// (declared in its tests/host_stubs/acl/acl.h:27-45), implemented over the CUDA
// runtime, so those harnesses (Session / Buffer / Events in
// tests/npu/turboquant_npu_common.hpp:326-380) build and run unmodified against
// libtq_b200.so. An aclrtStream is a cudaStream_t, an aclrtEvent a cudaEvent_t;
// enum arguments arrive as ints. Nothing here touches device settings.
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace {
inline int rc(cudaError_t e) { return e == cudaSuccess ? 0 : static_cast<int>(e); }
}

extern "C" {

int aclInit(const char*) { return 0; }
int aclFinalize() { return 0; }
int aclrtSetDevice(int device) { return rc(cudaSetDevice(device)); }
// The harness calls this on teardown; waiting for the device is all it needs.
int aclrtResetDevice(int) { return rc(cudaDeviceSynchronize()); }
int aclrtCreateStream(void** stream)
{
    cudaStream_t s = nullptr;
    const cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    *stream = s;
    return rc(e);
}
int aclrtDestroyStream(void* stream) { return rc(cudaStreamDestroy(static_cast<cudaStream_t>(stream))); }
int aclrtSynchronizeStream(void* stream)
{
    return rc(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
}
int aclrtMalloc(void** ptr, size_t size, int /*policy*/) { return rc(cudaMalloc(ptr, size)); }
int aclrtFree(void* ptr) { return rc(cudaFree(ptr)); }
int aclrtMemcpy(void* dst, size_t dst_max, const void* src, size_t count, int kind)
{
    if (count > dst_max) return static_cast<int>(cudaErrorInvalidValue);
    static const cudaMemcpyKind kinds[4] = {cudaMemcpyHostToHost, cudaMemcpyHostToDevice,
                                            cudaMemcpyDeviceToHost, cudaMemcpyDeviceToDevice};
    if (kind < 0 || kind > 3) return static_cast<int>(cudaErrorInvalidValue);
    // Blocking, like aclrtMemcpy: the harness reads results right after it returns.
    const cudaError_t e = cudaMemcpy(dst, src, count, kinds[kind]);
    return rc(e);
}
int aclrtMemset(void* ptr, size_t max_count, int32_t value, size_t count)
{
    if (count > max_count) return static_cast<int>(cudaErrorInvalidValue);
    const cudaError_t e = cudaMemset(ptr, value, count);
    if (e != cudaSuccess) return rc(e);
    return rc(cudaDeviceSynchronize());
}
int aclrtCreateEvent(void** event)
{
    cudaEvent_t ev = nullptr;
    const cudaError_t e = cudaEventCreate(&ev);
    *event = ev;
    return rc(e);
}
int aclrtDestroyEvent(void* event) { return rc(cudaEventDestroy(static_cast<cudaEvent_t>(event))); }
int aclrtRecordEvent(void* event, void* stream)
{
    return rc(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
}
int aclrtSynchronizeEvent(void* event) { return rc(cudaEventSynchronize(static_cast<cudaEvent_t>(event))); }
int aclrtEventElapsedTime(float* ms, void* start, void* end)
{
    return rc(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(end)));
}

}  // extern "C"
