// Device / buffer handles and error plumbing of the C ABI
// (the part of the boundary that mirrors ironmill-metal-sys device.rs / buffer.rs).
#include <stdarg.h>
#include <stdlib.h>

#include <new>

#include "common.cuh"

namespace im {

std::string &last_error() {
    static thread_local std::string msg;
    return msg;
}

int fail(int code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    last_error() = buf;
    return code;
}

int dev_malloc(Device *dev, void **ptr, size_t bytes) {
    *ptr = nullptr;
    if (bytes == 0) return IM_OK;
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(IM_ERR_ALLOC, "cudaMalloc(%zu bytes) failed: %s", bytes, cudaGetErrorString(e));
    }
    if (dev) dev->allocated += bytes;
    return IM_OK;
}

void dev_free(Device *dev, void *ptr, size_t bytes) {
    if (!ptr) return;
    cudaFree(ptr);
    if (dev && dev->allocated >= bytes) dev->allocated -= bytes;
}

}  // namespace im

struct im_buffer {
    im_device *dev;
    void *ptr;
    size_t bytes;
};

IM_EXPORT const char *im_cuda_last_error(void) { return im::last_error().c_str(); }
IM_EXPORT int im_cuda_abi_version(void) { return 1; }

IM_EXPORT int im_cuda_device_count(int *count_out) {
    IM_REQUIRE(count_out, "count_out is NULL");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *count_out = 0;
        return im::fail(IM_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    }
    *count_out = n;
    return IM_OK;
}

IM_EXPORT int im_cuda_device_open(int ordinal, im_device **out) {
    IM_GUARD_BEGIN
    IM_REQUIRE(out, "out is NULL");
    *out = nullptr;
    int n = 0;
    int rc = im_cuda_device_count(&n);
    if (rc != IM_OK) return rc;
    if (ordinal < 0 || ordinal >= n) return im::fail(IM_ERR_NO_DEVICE, "device ordinal %d out of range (%d devices)", ordinal, n);
    IM_CUDA_CHECK(cudaSetDevice(ordinal));
    im_device *d = new im_device();
    d->ordinal = ordinal;
    cudaError_t e = cudaGetDeviceProperties(&d->prop, ordinal);
    if (e != cudaSuccess) {
        delete d;
        return im::fail(IM_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    }
    d->sm_count = d->prop.multiProcessorCount;
    d->smem_optin = d->prop.sharedMemPerBlockOptin;
    if (d->prop.major != 10) {
        int major = d->prop.major, minor = d->prop.minor;
        delete d;
        return im::fail(IM_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", ordinal, major, minor);
    }
    // scratch of the tiled matvec (see common.cuh) and the device-side error word
    rc = im::dev_malloc(d, (void **)&d->sk_partial, (size_t)d->sm_count * 2 * 64 * sizeof(float));
    if (rc == IM_OK) rc = im::dev_malloc(d, (void **)&d->sk_counters, (size_t)im::kSkMaxBlocks * sizeof(int));
    if (rc == IM_OK) rc = im::dev_malloc(d, (void **)&d->err_flag, sizeof(int));
    if (rc == IM_OK) rc = im::dev_malloc(d, (void **)&d->gemm_partial, im::kGemmPartialBytes);
    if (rc == IM_OK && (cudaMemset(d->sk_counters, 0, (size_t)im::kSkMaxBlocks * sizeof(int)) != cudaSuccess ||
                        cudaMemset(d->err_flag, 0, sizeof(int)) != cudaSuccess))
        rc = im::fail(IM_ERR_CUDA, "scratch initialisation failed");
    if (rc != IM_OK) {
        im_cuda_device_free(d);
        return rc;
    }
    *out = d;
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT void im_cuda_device_free(im_device *dev) {
    if (!dev) return;
    cudaFree(dev->sk_partial);
    cudaFree(dev->sk_counters);
    cudaFree(dev->err_flag);
    cudaFree(dev->gemm_partial);
    delete dev;
}

IM_EXPORT int im_cuda_device_check_error(im_device *dev) {
    IM_REQUIRE(dev, "dev is NULL");
    int flag = 0;
    IM_CUDA_CHECK(cudaMemcpy(&flag, dev->err_flag, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag) {
        cudaMemset(dev->err_flag, 0, sizeof(int));
        cudaMemset(dev->sk_counters, 0, (size_t)im::kSkMaxBlocks * sizeof(int));
        return im::fail(IM_ERR_TIMEOUT, "a device-side bounded wait ran out; the results of the affected launch are invalid");
    }
    return IM_OK;
}
IM_EXPORT int im_cuda_device_ordinal(const im_device *dev) { return dev ? dev->ordinal : -1; }
IM_EXPORT int im_cuda_device_sm_count(const im_device *dev) { return dev ? dev->sm_count : 0; }
IM_EXPORT size_t im_cuda_device_allocated_bytes(const im_device *dev) { return dev ? dev->allocated : 0; }

IM_EXPORT int im_cuda_device_name(const im_device *dev, char *buf, size_t buf_len) {
    IM_REQUIRE(dev && buf && buf_len > 0, "bad argument");
    snprintf(buf, buf_len, "%s", dev->prop.name);
    return IM_OK;
}

IM_EXPORT int im_cuda_device_synchronize(im_device *dev) {
    IM_REQUIRE(dev, "dev is NULL");
    IM_CUDA_CHECK(cudaSetDevice(dev->ordinal));
    IM_CUDA_CHECK(cudaDeviceSynchronize());
    return IM_OK;
}

IM_EXPORT int im_cuda_buffer_alloc(im_device *dev, size_t bytes, im_buffer **out) {
    IM_GUARD_BEGIN
    IM_REQUIRE(dev && out, "bad argument");
    *out = nullptr;
    IM_REQUIRE(bytes > 0, "buffer size must be > 0");
    IM_CUDA_CHECK(cudaSetDevice(dev->ordinal));
    void *p = nullptr;
    int rc = im::dev_malloc(dev, &p, bytes);
    if (rc != IM_OK) return rc;
    *out = new im_buffer{dev, p, bytes};
    return IM_OK;
    IM_GUARD_END
}

IM_EXPORT int im_cuda_buffer_alloc_with_data(im_device *dev, const void *src_host, size_t bytes, im_buffer **out) {
    IM_REQUIRE(src_host, "src_host is NULL");
    int rc = im_cuda_buffer_alloc(dev, bytes, out);
    if (rc != IM_OK) return rc;
    rc = im_cuda_buffer_upload(*out, 0, src_host, bytes);
    if (rc != IM_OK) {
        im_cuda_buffer_free(*out);
        *out = nullptr;
    }
    return rc;
}

IM_EXPORT void im_cuda_buffer_free(im_buffer *buf) {
    if (!buf) return;
    im::dev_free(buf->dev, buf->ptr, buf->bytes);
    delete buf;
}

IM_EXPORT size_t im_cuda_buffer_length(const im_buffer *buf) { return buf ? buf->bytes : 0; }
IM_EXPORT void *im_cuda_buffer_ptr(const im_buffer *buf) { return buf ? buf->ptr : nullptr; }

IM_EXPORT int im_cuda_buffer_upload(im_buffer *buf, size_t offset, const void *src_host, size_t bytes) {
    IM_REQUIRE(buf && src_host, "bad argument");
    if (offset > buf->bytes || bytes > buf->bytes - offset)
        return im::fail(IM_ERR_BOUNDS, "upload of %zu bytes at offset %zu exceeds buffer length %zu", bytes, offset, buf->bytes);
    IM_CUDA_CHECK(cudaMemcpy(static_cast<char *>(buf->ptr) + offset, src_host, bytes, cudaMemcpyHostToDevice));
    return IM_OK;
}

IM_EXPORT int im_cuda_buffer_download(const im_buffer *buf, size_t offset, void *dst_host, size_t bytes) {
    IM_REQUIRE(buf && dst_host, "bad argument");
    if (offset > buf->bytes || bytes > buf->bytes - offset)
        return im::fail(IM_ERR_BOUNDS, "download of %zu bytes at offset %zu exceeds buffer length %zu", bytes, offset, buf->bytes);
    IM_CUDA_CHECK(cudaMemcpy(dst_host, static_cast<const char *>(buf->ptr) + offset, bytes, cudaMemcpyDeviceToHost));
    return IM_OK;
}
