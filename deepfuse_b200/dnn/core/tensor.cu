// dnn::tensor<TT> bodies.  Upstream counterpart: dnn/core/tensor.cu and dnn/core/tensor_transpose.cu.
#include "dnn/core/tensor.cuh"

#include <algorithm>
#include <cmath>
#include <numeric>
#include <sstream>
#include <stdexcept>
#include <type_traits>

#include "dnn/core/cuda.cuh"
#include "dnn/utils/common.cuh"

namespace dnn {

namespace {

constexpr int kBlock = 256;

inline int grid_for(size_t n) {
    size_t g = (n + kBlock - 1) / kBlock;
    return int(std::min<size_t>(std::max<size_t>(g, 1), 148 * 16));
}

template <typename TT>
__device__ __forceinline__ float as_float(TT v) {
    if constexpr (std::is_same_v<TT, __half>) return __half2float(v);
    else if constexpr (std::is_same_v<TT, __nv_bfloat16>) return __bfloat162float(v);
    else return static_cast<float>(v);
}

template <typename TT>
__device__ __forceinline__ TT from_float(float v) {
    if constexpr (std::is_same_v<TT, __half>) return __float2half(v);
    else if constexpr (std::is_same_v<TT, __nv_bfloat16>) return __float2bfloat16(v);
    else return static_cast<TT>(v);
}

template <typename TT>
__global__ void fill_kernel(TT* p, size_t n, TT v) {
    for (size_t i = blockIdx.x * size_t(kBlock) + threadIdx.x; i < n; i += size_t(gridDim.x) * kBlock) p[i] = v;
}

// out = a + b; floating types add in fp32 and round once, integers add natively
template <typename TT>
__global__ void add_kernel(const TT* a, const TT* b, TT* out, size_t n) {
    for (size_t i = blockIdx.x * size_t(kBlock) + threadIdx.x; i < n; i += size_t(gridDim.x) * kBlock) {
        if constexpr (std::is_integral_v<TT>) out[i] = TT(a[i] + b[i]);
        else out[i] = from_float<TT>(as_float(a[i]) + as_float(b[i]));
    }
}

template <typename TT>
__global__ void equal_mask_kernel(const TT* a, const TT* b, uint8_t* out, size_t n) {
    for (size_t i = blockIdx.x * size_t(kBlock) + threadIdx.x; i < n; i += size_t(gridDim.x) * kBlock)
        out[i] = as_float(a[i]) == as_float(b[i]) ? 1 : 0;
}

// counts positions where |a-b| > atol (atol < 0: bitwise inequality)
template <typename TT>
__global__ void mismatch_count_kernel(const TT* a, const TT* b, size_t n, float atol, unsigned long long* count) {
    unsigned long long local = 0;
    for (size_t i = blockIdx.x * size_t(kBlock) + threadIdx.x; i < n; i += size_t(gridDim.x) * kBlock) {
        bool bad;
        if (atol < 0.f) {
            const unsigned char* pa = reinterpret_cast<const unsigned char*>(a + i);
            const unsigned char* pb = reinterpret_cast<const unsigned char*>(b + i);
            bad = false;
            for (int k = 0; k < int(sizeof(TT)); ++k) bad |= pa[k] != pb[k];
        } else {
            const float d = fabsf(as_float(a[i]) - as_float(b[i]));
            bad = !(d <= atol);
        }
        local += bad ? 1 : 0;
    }
    if (local) atomicAdd(count, local);
}

// generic strided gather: out (dense, `rank` dims of out_shape) <- in at sum(idx[d] * in_stride[d]) + offset
struct GatherDesc {
    int rank;
    int out_shape[8];
    long long in_stride[8];
    long long offset;
};

template <typename TT>
__global__ void gather_kernel(const TT* in, TT* out, size_t n, GatherDesc d) {
    for (size_t i = blockIdx.x * size_t(kBlock) + threadIdx.x; i < n; i += size_t(gridDim.x) * kBlock) {
        size_t rem = i;
        long long src = d.offset;
        for (int k = d.rank - 1; k >= 0; --k) {
            const int c = int(rem % size_t(d.out_shape[k]));
            rem /= size_t(d.out_shape[k]);
            src += c * d.in_stride[k];
        }
        out[i] = in[src];
    }
}

size_t count_of(const std::vector<int>& shape) {
    size_t n = 1;
    for (int s : shape) {
        if (s < 0) throw std::invalid_argument("tensor: negative dimension");
        n *= size_t(s);
    }
    return n;
}

std::string shape_text(const std::vector<int>& s) {
    std::ostringstream os;
    os << "[";
    for (size_t i = 0; i < s.size(); ++i) os << (i ? ", " : "") << s[i];
    os << "]";
    return os.str();
}

template <typename TT>
TT* pool_alloc(size_t n) {
    if (n == 0) return nullptr;
    void* p = nullptr;
    utils::CHECK_CUDA_EX(cudaMallocAsync(&p, n * sizeof(TT), Cuda::stream()));
    return static_cast<TT*>(p);
}

inline void pool_free(void* p) {
    if (p) cudaFreeAsync(p, Cuda::stream());
}

}  // namespace

template <typename TT>
tensor<TT>::tensor(const std::vector<int>& shape) : shape_(shape), total_size_(count_of(shape)) {
    if (total_size_ > size_t(0x7fffffff)) throw std::invalid_argument("tensor: more than 2^31-1 elements");
    data_ = pool_alloc<TT>(total_size_);
}

template <typename TT>
tensor<TT>::~tensor() {
    pool_free(data_);
}

template <typename TT>
tensor<TT>::tensor(tensor&& o) noexcept
    : shape_(std::move(o.shape_)), data_(o.data_), total_size_(o.total_size_), version_(o.version_ + 1) {
    o.data_ = nullptr;
    o.total_size_ = 0;
    o.shape_.clear();
}

template <typename TT>
tensor<TT>& tensor<TT>::operator=(tensor&& o) noexcept {
    if (this != &o) {
        pool_free(data_);
        shape_ = std::move(o.shape_);
        data_ = o.data_;
        total_size_ = o.total_size_;
        version_ += o.version_ + 1;  // strictly increases for this object: the content was replaced
        o.data_ = nullptr;
        o.total_size_ = 0;
        o.shape_.clear();
    }
    return *this;
}

template <typename TT>
void tensor<TT>::upload(const TT* host_data) {
    if (total_size_)
        utils::CHECK_CUDA_EX(
            cudaMemcpyAsync(data_, host_data, total_size_ * sizeof(TT), cudaMemcpyHostToDevice, Cuda::stream()));
    // pageable sources are staged before the call returns; pinned sources must outlive the copy
    ++version_;
}

template <typename TT>
void tensor<TT>::download(TT* host_data) const {
    if (total_size_)
        utils::CHECK_CUDA_EX(
            cudaMemcpyAsync(host_data, data_, total_size_ * sizeof(TT), cudaMemcpyDeviceToHost, Cuda::stream()));
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
    // results reach the host here: if a bounded device-side wait of the kernel library gave up on the way, the
    // data is incomplete, and the caller gets the exception a failed CUDA call would raise
    utils::CHECK_DF8(df8_status_word_check());
}

template <typename TT>
int tensor<TT>::size(int dim) const {
    if (dim < 0 || dim >= int(shape_.size()))
        throw std::out_of_range("tensor::size: dimension " + std::to_string(dim) + " out of range for shape " +
                                shape_text(shape_));
    return shape_[size_t(dim)];
}

template <typename TT>
tensor<TT>& tensor<TT>::reshape(const std::vector<int>& new_shape) {
    if (count_of(new_shape) != total_size_)
        throw std::runtime_error("tensor::reshape: cannot view " + shape_text(shape_) + " as " +
                                 shape_text(new_shape));
    shape_ = new_shape;
    return *this;
}

template <typename TT>
tensor<TT>& tensor<TT>::fill(TT value) {
    if (total_size_) {
        fill_kernel<TT><<<grid_for(total_size_), kBlock, 0, Cuda::stream()>>>(data_, total_size_, value);
        utils::THROW_CUDA_EX();
    }
    ++version_;
    return *this;
}

template <typename TT>
tensor<TT>& tensor<TT>::zero() {
    if (total_size_) utils::CHECK_CUDA_EX(cudaMemsetAsync(data_, 0, total_size_ * sizeof(TT), Cuda::stream()));
    ++version_;
    return *this;
}

template <typename TT>
tensor<TT> tensor<TT>::clone() const {
    tensor<TT> out(shape_);
    if (total_size_)
        utils::CHECK_CUDA_EX(
            cudaMemcpyAsync(out.data_, data_, total_size_ * sizeof(TT), cudaMemcpyDeviceToDevice, Cuda::stream()));
    return out;
}

template <typename TT>
tensor<TT>& tensor<TT>::operator+=(const tensor<TT>& other) {
    if (shape_ != other.shape_)
        throw std::runtime_error("tensor::operator+=: shape mismatch " + shape_text(shape_) + " vs " +
                                 shape_text(other.shape_));
    if (total_size_) {
        add_kernel<TT><<<grid_for(total_size_), kBlock, 0, Cuda::stream()>>>(data_, other.data_, data_, total_size_);
        utils::THROW_CUDA_EX();
    }
    ++version_;
    return *this;
}

template <typename TT>
tensor<TT> operator+(const tensor<TT>& a, const tensor<TT>& b) {
    if (a.shape() != b.shape())
        throw std::runtime_error("tensor operator+: shape mismatch " + shape_text(a.shape()) + " vs " +
                                 shape_text(b.shape()));
    tensor<TT> out(a.shape());
    if (a.numel()) {
        add_kernel<TT><<<grid_for(a.numel()), kBlock, 0, Cuda::stream()>>>(a.data(), b.data(), out.data(), a.numel());
        utils::THROW_CUDA_EX();
    }
    return out;
}

template <typename TT>
tensor<uint8_t> tensor<TT>::operator==(const tensor<TT>& other) const {
    if (shape_ != other.shape_)
        throw std::runtime_error("tensor::operator==: shape mismatch " + shape_text(shape_) + " vs " +
                                 shape_text(other.shape_));
    tensor<uint8_t> out(shape_);
    if (total_size_) {
        equal_mask_kernel<TT><<<grid_for(total_size_), kBlock, 0, Cuda::stream()>>>(data_, other.data_, out.data(),
                                                                                   total_size_);
        utils::THROW_CUDA_EX();
    }
    return out;
}

namespace {
template <typename TT>
bool compare(const tensor<TT>& a, const tensor<TT>& b, float atol) {
    if (a.shape() != b.shape()) return false;
    if (a.numel() == 0) return true;
    tensor<int> scratch({2});  // 8 bytes, used as one 64-bit counter
    unsigned long long* count = reinterpret_cast<unsigned long long*>(scratch.data());
    utils::CHECK_CUDA_EX(cudaMemsetAsync(count, 0, sizeof(unsigned long long), Cuda::stream()));
    mismatch_count_kernel<TT><<<grid_for(a.numel()), kBlock, 0, Cuda::stream()>>>(a.data(), b.data(), a.numel(), atol,
                                                                                 count);
    utils::THROW_CUDA_EX();
    unsigned long long host = 0;
    utils::CHECK_CUDA_EX(cudaMemcpyAsync(&host, count, sizeof(host), cudaMemcpyDeviceToHost, Cuda::stream()));
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
    return host == 0;
}
}  // namespace

template <typename TT>
bool tensor<TT>::equals(const tensor<TT>& other) const {
    return compare(*this, other, -1.0f);
}

template <typename TT>
bool tensor<TT>::approx_equal(const tensor<TT>& other, float atol) const {
    return compare(*this, other, atol);
}

template <typename TT>
tensor<TT>& tensor<TT>::narrow(int dim, int start, int length) {
    const int rank = int(shape_.size());
    if (dim < 0 || dim >= rank || start < 0 || length <= 0 || start + length > shape_[size_t(dim)])
        throw std::invalid_argument("tensor::narrow: bad arguments (dim " + std::to_string(dim) + ", start " +
                                    std::to_string(start) + ", length " + std::to_string(length) + ") for shape " +
                                    shape_text(shape_));
    if (rank > 8) throw std::invalid_argument("tensor::narrow: rank above 8");
    std::vector<int> out_shape = shape_;
    out_shape[size_t(dim)] = length;
    GatherDesc d{};
    d.rank = rank;
    long long stride = 1;
    for (int k = rank - 1; k >= 0; --k) {
        d.out_shape[k] = out_shape[size_t(k)];
        d.in_stride[k] = stride;
        stride *= shape_[size_t(k)];
    }
    d.offset = (long long)start * d.in_stride[dim];
    const size_t n = count_of(out_shape);
    TT* fresh = pool_alloc<TT>(n);
    if (n) {
        gather_kernel<TT><<<grid_for(n), kBlock, 0, Cuda::stream()>>>(data_, fresh, n, d);
        utils::THROW_CUDA_EX();
    }
    pool_free(data_);
    data_ = fresh;
    shape_ = out_shape;
    total_size_ = n;
    ++version_;
    return *this;
}

template <typename TT>
tensor<TT>& tensor<TT>::slice(int dim, int start, int end) {
    if (end <= start) throw std::invalid_argument("tensor::slice: end must be greater than start");
    return narrow(dim, start, end - start);
}

template <typename TT>
tensor<TT>& tensor<TT>::permute(const std::vector<int>& perm) {
    const int rank = int(shape_.size());
    if (int(perm.size()) != rank || rank > 8) throw std::invalid_argument("tensor::permute: bad permutation length");
    std::vector<bool> seen(size_t(rank), false);
    for (int p : perm) {
        if (p < 0 || p >= rank || seen[size_t(p)]) throw std::invalid_argument("tensor::permute: not a permutation");
        seen[size_t(p)] = true;
    }
    std::vector<long long> in_stride(size_t(rank), 1);
    for (int k = rank - 2; k >= 0; --k) in_stride[size_t(k)] = in_stride[size_t(k) + 1] * shape_[size_t(k) + 1];
    GatherDesc d{};
    d.rank = rank;
    std::vector<int> out_shape(size_t(rank), 0);
    for (int k = 0; k < rank; ++k) {
        out_shape[size_t(k)] = shape_[size_t(perm[size_t(k)])];
        d.out_shape[k] = out_shape[size_t(k)];
        d.in_stride[k] = in_stride[size_t(perm[size_t(k)])];
    }
    d.offset = 0;
    TT* fresh = pool_alloc<TT>(total_size_);
    if (total_size_) {
        gather_kernel<TT><<<grid_for(total_size_), kBlock, 0, Cuda::stream()>>>(data_, fresh, total_size_, d);
        utils::THROW_CUDA_EX();
    }
    pool_free(data_);
    data_ = fresh;
    shape_ = out_shape;
    ++version_;
    return *this;
}

// Swaps the channel-first and channel-last layouts of a 4-D tensor (N kept in front), and plainly
// transposes a 2-D one.
template <typename TT>
tensor<TT>& tensor<TT>::transpose() {
    if (shape_.size() == 2) return permute({1, 0});
    if (shape_.size() == 4) return permute({0, 2, 3, 1});
    throw std::invalid_argument("tensor::transpose: only 2-D and 4-D tensors");
}

template <typename TT>
std::string tensor<TT>::to_string() const {
    std::ostringstream os;
    os << "tensor" << shape_text(shape_);
    const size_t show = std::min<size_t>(total_size_, 16);
    if (show) {
        std::vector<TT> host(total_size_);
        download(host.data());
        os << " {";
        for (size_t i = 0; i < show; ++i) {
            float v;
            if constexpr (std::is_same_v<TT, __half>) v = __half2float(host[i]);
            else if constexpr (std::is_same_v<TT, __nv_bfloat16>) v = __bfloat162float(host[i]);
            else v = float(host[i]);
            os << (i ? ", " : "") << v;
        }
        os << (show < total_size_ ? ", ...}" : "}");
    }
    return os.str();
}

template <typename TT>
void tensor<TT>::save(std::ostream& out) const {
    const int ndim = int(shape_.size());
    out.write(reinterpret_cast<const char*>(&ndim), sizeof(ndim));
    out.write(reinterpret_cast<const char*>(shape_.data()), std::streamsize(sizeof(int)) * ndim);
    std::vector<TT> host(total_size_);
    download(host.data());
    out.write(reinterpret_cast<const char*>(host.data()), std::streamsize(sizeof(TT) * total_size_));
}

template <typename TT>
void tensor<TT>::load(std::istream& in) {
    int ndim = 0;
    in.read(reinterpret_cast<char*>(&ndim), sizeof(ndim));
    if (!in || ndim < 0 || ndim > 8) throw std::runtime_error("tensor::load: bad header");
    std::vector<int> shape(size_t(ndim), 0);
    in.read(reinterpret_cast<char*>(shape.data()), std::streamsize(sizeof(int)) * ndim);
    if (!in) throw std::runtime_error("tensor::load: truncated shape");
    tensor<TT> fresh(shape);
    std::vector<TT> host(fresh.numel());
    in.read(reinterpret_cast<char*>(host.data()), std::streamsize(sizeof(TT) * host.size()));
    if (!in) throw std::runtime_error("tensor::load: truncated data");
    fresh.upload(host.data());
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));  // `host` dies at scope exit
    *this = std::move(fresh);
}

#define DNN_INSTANTIATE_TENSOR(T)   \
    template struct tensor<T>;      \
    template tensor<T> operator+ <T>(const tensor<T>&, const tensor<T>&);

DNN_INSTANTIATE_TENSOR(float)
DNN_INSTANTIATE_TENSOR(__half)
DNN_INSTANTIATE_TENSOR(__nv_bfloat16)
DNN_INSTANTIATE_TENSOR(int)
DNN_INSTANTIATE_TENSOR(int8_t)
DNN_INSTANTIATE_TENSOR(uint8_t)

}  // namespace dnn
