// dnn::tensor<TT> — move-only owner of a dense row-major device buffer plus its shape.
//
// Public surface of upstream dnn/core/tensor.cuh:23-149 (constructor from a shape, upload/download,
// data, shape, size, size(dim), reshape, fill, zero, clone, +=, ==, equals, approx_equal,
// narrow, slice, transpose, permute, to_string, save, load, operator+ and the tensorf/... aliases),
// with upstream's error behaviour (dnn/core/tensor.cu:211-243, :385-387, :403-405, :420-423).
//
// What differs underneath:
//  * memory comes from the device's stream-ordered pool (cudaMallocAsync on Cuda::stream()), so the
//    value-returning forward() of every layer does not pay a cudaMalloc/cudaFree pair and an implicit
//    device synchronisation per temporary as upstream's constructor/destructor do (tensor.cu:92,178);
//  * every operation is enqueued on Cuda::stream(); only download(), equals() and approx_equal()
//    wait for the stream, because they return host data;
//  * element counts are kept as size_t internally; size() still returns int as upstream does;
//  * version() counts content changes made through this API, which lets a layer notice that its fp32
//    weights were re-uploaded and re-quantise its cached fp8 copy.
// fp8 values are stored as raw codes in tensor<uint8_t> (tensoru8).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <iostream>
#include <string>
#include <vector>

namespace dnn {

template <typename TT>
struct tensor {
protected:
    std::vector<int> shape_;
    TT* data_ = nullptr;
    size_t total_size_ = 0;
    uint64_t version_ = 0;

public:
    tensor(const std::vector<int>& shape);  // implicit, as upstream's (core/tensor.cuh:34)
    virtual ~tensor();

    tensor(const tensor&) = delete;
    tensor& operator=(const tensor&) = delete;
    tensor(tensor&& other) noexcept;
    tensor& operator=(tensor&& other) noexcept;

    // host -> device / device -> host copies of size() elements
    virtual void upload(const TT* host_data);
    virtual void download(TT* host_data) const;

    TT* data() { return data_; }
    const TT* data() const { return data_; }
    const std::vector<int>& shape() const { return shape_; }
    int size() const { return static_cast<int>(total_size_); }
    size_t numel() const { return total_size_; }
    int size(int dim) const;  // throws std::out_of_range
    uint64_t version() const { return version_; }
    void bump_version() { ++version_; }  // call after writing through data()

    tensor<TT>& reshape(const std::vector<int>& new_shape);  // metadata only; throws on size mismatch
    tensor<TT>& fill(TT value);
    tensor<TT>& zero();
    tensor<TT> clone() const;

    tensor<TT>& operator+=(const tensor<TT>& other);
    tensor<uint8_t> operator==(const tensor<TT>& other) const;
    bool equals(const tensor<TT>& other) const;
    bool approx_equal(const tensor<TT>& other, float atol = 1e-5f) const;

    tensor<TT>& narrow(int dim, int start, int length);
    tensor<TT>& slice(int dim, int start, int end);
    tensor<TT>& transpose();
    tensor<TT>& permute(const std::vector<int>& perm);

    std::string to_string() const;

    // binary layout shared with upstream: int ndim, int shape[ndim], raw elements
    void save(std::ostream& out) const;
    void load(std::istream& in);
};

template <typename TT>
tensor<TT> operator+(const tensor<TT>& a, const tensor<TT>& b);

using tensorf = tensor<float>;
using tensorh = tensor<__half>;
using tensorbf = tensor<__nv_bfloat16>;
using tensori = tensor<int>;
using tensori8 = tensor<int8_t>;
using tensoru8 = tensor<uint8_t>;

}  // namespace dnn
