// What a step moves between the host and the device, with as little host time per call as the runtime allows:
// one asynchronous copy of the step's descriptors with an event recorded behind it, and the address under which
// kernels write into page-locked host memory.  No kernels here.
#include "common.cuh"

// The address under which kernels of the current device reach pinned (page-locked) host memory, or null if they
// cannot: the sampler writes its few tokens straight to the host through it, sparing a copy per step.
VM_API void* vm_host_device_pointer(void* host) {
    void* dev = nullptr;
    if (cudaHostGetDevicePointer(&dev, host, 0) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return dev;
}

// An event without timing, for "has this copy left the host buffer": null on failure.
VM_API void* vm_event_create() {
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return e;
}

VM_API int vm_event_destroy(void* event) { return (int)cudaEventDestroy(static_cast<cudaEvent_t>(event)); }

VM_API int vm_event_synchronize(void* event) { return (int)cudaEventSynchronize(static_cast<cudaEvent_t>(event)); }

// dst (device) <- src (pinned host), nbytes, on `stream`; `event` (may be null) is recorded behind the copy.
VM_API int vm_upload_record(void* dst, const void* src, long long nbytes, void* event, cudaStream_t stream) {
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return (int)e;
    if (event != nullptr) e = cudaEventRecord(static_cast<cudaEvent_t>(event), stream);
    return (int)e;
}
