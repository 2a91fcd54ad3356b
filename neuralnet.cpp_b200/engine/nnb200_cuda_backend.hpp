// Stand-in for the reference's backend/cuda_backend.hpp: the same classes (CudaBuffer, CudaTensor,
// CudaBackend) with the same public members the rest of the reference uses (tensor.hpp:60-175,
// cli/engine_factory.hpp:50-58), on top of the C ABI of libnnb200 instead of the CUDA runtime and
// cuBLAS.  It defines the reference header's include guard, so a translation unit that force-includes
// this file first (-include) compiles the unchanged reference sources against it:
//
//   g++ -std=gnu++23 -DNN_HAS_CUDA -I<reference>/include -I<this repo>/include \
//       -include nnb200_cuda_backend.hpp -include nnb200_cuda_engine.hpp  prog.cpp  -lnnb200
//
// What differs from the reference backend, by design:
//   - device memory comes from a stream-ordered pool (nnb200_rt_alloc / nnb200_rt_free), not a
//     cudaMalloc / cudaFree pair around every op output;
//   - the device is LOCAL_RANK (one process per GPU) rather than always device 0;
//   - the per-op *_gpu members are gone: CudaEngine calls the C ABI directly.
#ifndef NN_CUDA_BACKEND_HPP
#define NN_CUDA_BACKEND_HPP
#ifdef NN_HAS_CUDA

#include <cstddef>
#include <cstdint>
#include <memory>
#include <span>
#include <string>

#include "neuralnet.cpp/algebra_matrix.hpp"
#include "neuralnet.cpp/config.hpp"
#include "neuralnet.cpp/core_errors.hpp"
#include "nnb200.h"

namespace nn
{

namespace cuda_detail
{
// 0 -> success; anything else -> Error naming the entry point and the code it returned
[[nodiscard]] inline Result<void> check(int rc, const char* what)
{
    if (rc == 0) return {};
    return std::unexpected(Error{std::string(what) + " failed (code " + std::to_string(rc) + ")"});
}
} // namespace cuda_detail

// Owns one block of the runtime's memory pool; `size` counts floats (backend/cuda_backend.hpp:66-122).
class CudaBuffer
{
private:
    void* ptr_ = nullptr;
    std::size_t size_ = 0;
    bool owned_ = true;             // false: a view into memory another buffer owns (see borrowed())

    void release() noexcept
    {
        if (ptr_ && owned_) (void)nnb200_rt_free(ptr_);
        ptr_ = nullptr;
        size_ = 0;
        owned_ = true;
    }

public:
    CudaBuffer() = default;
    CudaBuffer(void* ptr, std::size_t size) : ptr_(ptr), size_(size) {}
    ~CudaBuffer() { release(); }
    CudaBuffer(CudaBuffer&& o) noexcept : ptr_(o.ptr_), size_(o.size_), owned_(o.owned_) { o.ptr_ = nullptr; o.size_ = 0; }
    CudaBuffer& operator=(CudaBuffer&& o) noexcept
    {
        if (this != &o)
        {
            release();
            ptr_ = o.ptr_;
            size_ = o.size_;
            owned_ = o.owned_;
            o.ptr_ = nullptr;
            o.size_ = 0;
        }
        return *this;
    }
    CudaBuffer(const CudaBuffer&) = delete;
    CudaBuffer& operator=(const CudaBuffer&) = delete;

    [[nodiscard]] static Result<CudaBuffer> allocate(std::size_t elem_count)
    {
        void* p = nullptr;
        // an empty tensor still gets a block, so that data() is a valid device address
        const std::size_t bytes = (elem_count ? elem_count : 1) * sizeof(float);
        if (const int rc = nnb200_rt_alloc(bytes, &p); rc != 0 || !p)
            return std::unexpected(Error{"device allocation failed (code " + std::to_string(rc) + ", " +
                                         std::to_string(bytes) + " bytes)"});
        return CudaBuffer(p, elem_count);
    }

    // A non-owning buffer over `elem_count` floats at `ptr`: parameter and gradient tensors that are slices of one
    // arena (the fused GPT model) are built on these; the arena's own buffer frees the memory.
    [[nodiscard]] static CudaBuffer borrowed(void* ptr, std::size_t elem_count) noexcept
    {
        CudaBuffer b(ptr, elem_count);
        b.owned_ = false;
        return b;
    }

    [[nodiscard]] void* ptr() const noexcept { return ptr_; }
    [[nodiscard]] std::size_t size() const noexcept { return size_; }
    [[nodiscard]] bool valid() const noexcept { return ptr_ != nullptr; }
};

class CudaBackend;

// A (rows, cols) row-major fp32 view of a shared buffer (backend/cuda_backend.hpp:127-166).
class CudaTensor
{
private:
    std::shared_ptr<CudaBuffer> buffer_;
    std::size_t rows_ = 0;
    std::size_t cols_ = 0;

public:
    CudaTensor() = default;
    CudaTensor(std::shared_ptr<CudaBuffer> buffer, std::size_t rows, std::size_t cols)
        : buffer_(std::move(buffer)), rows_(rows), cols_(cols) {}

    [[nodiscard]] static Result<CudaTensor> from_matrix(const Matrix& cpu_mat, CudaBackend& backend);
    [[nodiscard]] static Result<CudaTensor> create_empty(std::size_t rows, std::size_t cols, CudaBackend& backend);
    [[nodiscard]] Result<Matrix> to_matrix(CudaBackend& backend) const;

    [[nodiscard]] std::size_t rows() const noexcept { return rows_; }
    [[nodiscard]] std::size_t cols() const noexcept { return cols_; }
    [[nodiscard]] bool valid() const noexcept { return buffer_ && buffer_->valid(); }
    [[nodiscard]] const CudaBuffer& buffer() const noexcept { return *buffer_; }
    [[nodiscard]] float* data() const noexcept { return buffer_ ? static_cast<float*>(buffer_->ptr()) : nullptr; }
    [[nodiscard]] CudaTensor with_shape(std::size_t new_rows, std::size_t new_cols) const
    {
        return CudaTensor(buffer_, new_rows, new_cols);
    }
};

// What engine_factory.hpp prints after initialize(); field names follow cudaDeviceProp.
struct CudaDeviceProps
{
    char name[256] = {};
    std::size_t totalGlobalMem = 0;
    int multiProcessorCount = 0;
};

// Process-wide device context (backend/cuda_backend.hpp:169-337).
class CudaBackend
{
private:
    bool initialized_ = false;
    bool in_batch_ = false;
    CudaDeviceProps props_{};

    CudaBackend() = default;

public:
    CudaBackend(const CudaBackend&) = delete;
    CudaBackend& operator=(const CudaBackend&) = delete;

    [[nodiscard]] static CudaBackend& instance()
    {
        static CudaBackend backend;
        return backend;
    }

    [[nodiscard]] Result<void> initialize()
    {
        if (initialized_) return {};
        const int rc = nnb200_rt_init(-1, props_.name, sizeof(props_.name), &props_.totalGlobalMem,
                                      &props_.multiProcessorCount);
        if (rc != 0)
            return std::unexpected(Error{"CUDA initialisation failed (code " + std::to_string(rc) + ")"});
        initialized_ = true;
        return {};
    }

    [[nodiscard]] bool is_initialized() const noexcept { return initialized_; }
    [[nodiscard]] bool gpu_available() const noexcept { return initialized_; }
    [[nodiscard]] const CudaDeviceProps& device_props() const noexcept { return props_; }
    [[nodiscard]] int device_id() const noexcept { return nnb200_rt_device(); }
    [[nodiscard]] void* stream_ptr() const noexcept { return nnb200_rt_stream(); }

    // Work is queued on one stream in program order, so a batch needs no bookkeeping: begin marks it,
    // end waits for the queue to drain.
    [[nodiscard]] Result<void> begin_batch()
    {
        in_batch_ = true;
        return {};
    }
    [[nodiscard]] Result<void> end_batch()
    {
        in_batch_ = false;
        return sync_stream();
    }
    [[nodiscard]] bool in_batch() const noexcept { return in_batch_; }
    [[nodiscard]] Result<void> sync_stream() { return cuda_detail::check(nnb200_rt_sync(), "stream synchronise"); }

    [[nodiscard]] Result<void> upload_blocking(CudaTensor& dst, std::span<const Scalar> cpu_data)
    {
        if (!dst.valid()) return std::unexpected(Error{"upload: invalid CudaTensor"});
        if (cpu_data.size() > dst.buffer().size()) return std::unexpected(Error{"upload: size exceeds the buffer"});
        return cuda_detail::check(nnb200_rt_upload(dst.data(), cpu_data.data(), cpu_data.size_bytes()), "upload");
    }
    [[nodiscard]] Result<void> download_blocking(const CudaTensor& src, std::span<Scalar> cpu_data)
    {
        if (!src.valid()) return std::unexpected(Error{"download: invalid CudaTensor"});
        if (cpu_data.size() > src.buffer().size()) return std::unexpected(Error{"download: size exceeds the buffer"});
        return cuda_detail::check(nnb200_rt_download(cpu_data.data(), src.data(), cpu_data.size_bytes()), "download");
    }
};

inline Result<CudaTensor> CudaTensor::from_matrix(const Matrix& cpu_mat, CudaBackend& backend)
{
    if (cpu_mat.empty()) return std::unexpected(Error{"Empty matrix"});
    auto t = create_empty(cpu_mat.rows(), cpu_mat.cols(), backend);
    if (!t) return std::unexpected(t.error());
    if (auto up = backend.upload_blocking(*t, cpu_mat.span()); !up) return std::unexpected(up.error());
    return t;
}

inline Result<CudaTensor> CudaTensor::create_empty(std::size_t rows, std::size_t cols, CudaBackend& backend)
{
    if (!backend.is_initialized()) return std::unexpected(Error{"CudaBackend is not initialised"});
    auto buf = CudaBuffer::allocate(rows * cols);
    if (!buf) return std::unexpected(buf.error());
    return CudaTensor(std::make_shared<CudaBuffer>(std::move(*buf)), rows, cols);
}

inline Result<Matrix> CudaTensor::to_matrix(CudaBackend& backend) const
{
    if (!valid()) return std::unexpected(Error{"Invalid CudaTensor"});
    Matrix cpu_mat(rows_, cols_);
    if (auto dl = backend.download_blocking(*this, cpu_mat.span()); !dl) return std::unexpected(dl.error());
    return cpu_mat;
}

} // namespace nn

#endif // NN_HAS_CUDA
#endif // NN_CUDA_BACKEND_HPP
