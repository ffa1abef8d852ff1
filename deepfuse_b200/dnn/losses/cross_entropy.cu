#include "dnn/losses/cross_entropy.cuh"

#include <stdexcept>
#include <vector>

#include "df8.h"
#include "dnn/core/cuda.cuh"
#include "dnn/core/fp8.cuh"
#include "dnn/utils/common.cuh"

namespace dnn {

namespace {
void check_indices() {
    unsigned int bad = 0;
    utils::CHECK_DF8(df8_cross_entropy_bad_indices(&bad, 1));
    if (bad) throw std::runtime_error("CrossEntropyLoss: " + std::to_string(bad) + " target index(es) outside [0, classes)");
}
template <typename T>
void rows_and_classes(const tensor<T>& logits, int* rows, int* classes) {
    const auto& s = logits.shape();
    if (s.empty() || logits.numel() == 0) throw std::runtime_error("CrossEntropyLoss: empty logits");
    *classes = s.back();
    *rows = int(logits.numel() / size_t(*classes));
}
}  // namespace

// upstream sums the row losses on the host, in row order, in a float (cross_entropy.cu:155-168)
template <typename T>
T CrossEntropyLoss<T>::mean_of_rows(const tensor<T>& row_loss) const {
    std::vector<T> h(row_loss.numel());
    row_loss.download(h.data());
    float sum = 0.0f;
    for (T v : h) sum += static_cast<float>(v);
    return static_cast<T>(sum / static_cast<float>(h.size()));
}

template <typename T>
T CrossEntropyLoss<T>::compute(const tensor<T>& logits, const tensor<T>& targets) {
    int rows = 0, C = 0;
    rows_and_classes(logits, &rows, &C);
    if (targets.numel() != logits.numel()) throw std::runtime_error("CrossEntropyLoss: targets must have the logits' shape");
    tensor<T> row_loss({rows});
    utils::CHECK_DF8(df8_cross_entropy_f32(logits.data(), C, targets.data(), C, nullptr, rows, C, row_loss.data(), fp8::stream()));
    return mean_of_rows(row_loss);
}

template <typename T>
tensor<T> CrossEntropyLoss<T>::compute_gradient(const tensor<T>& logits, const tensor<T>& targets) {
    int rows = 0, C = 0;
    rows_and_classes(logits, &rows, &C);
    if (targets.numel() != logits.numel()) throw std::runtime_error("CrossEntropyLoss: targets must have the logits' shape");
    tensor<T> grad(logits.shape());
    utils::CHECK_DF8(df8_cross_entropy_grad_f32(logits.data(), C, targets.data(), C, nullptr, rows, C, grad.data(), C, fp8::stream()));
    return grad;
}

template <typename T>
T CrossEntropyLoss<T>::compute(const tensor<T>& logits, const tensor<int>& idx) {
    int rows = 0, C = 0;
    rows_and_classes(logits, &rows, &C);
    if (idx.numel() != size_t(rows)) throw std::runtime_error("CrossEntropyLoss: one target index per row of the logits");
    tensor<T> row_loss({rows});
    utils::CHECK_DF8(df8_cross_entropy_f32(logits.data(), C, nullptr, 0, idx.data(), rows, C, row_loss.data(), fp8::stream()));
    const T mean = mean_of_rows(row_loss);  // the download orders the host behind the kernel
    check_indices();
    return mean;
}

template <typename T>
tensor<T> CrossEntropyLoss<T>::compute_gradient(const tensor<T>& logits, const tensor<int>& idx) {
    int rows = 0, C = 0;
    rows_and_classes(logits, &rows, &C);
    if (idx.numel() != size_t(rows)) throw std::runtime_error("CrossEntropyLoss: one target index per row of the logits");
    tensor<T> grad(logits.shape());
    utils::CHECK_DF8(df8_cross_entropy_grad_f32(logits.data(), C, nullptr, 0, idx.data(), rows, C, grad.data(), C, fp8::stream()));
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
    check_indices();
    return grad;
}

template <typename T>
T CrossEntropyLoss<T>::compute_pitched(const tensor<T>& logits, int classes, const tensor<int>& idx) {
    const auto& s = logits.shape();
    if (s.size() != 2 || classes <= 0 || s[1] < classes) throw std::runtime_error("CrossEntropyLoss::compute_pitched: logits must be [rows, pitch >= classes]");
    const int rows = s[0], pitch = s[1];
    if (idx.numel() != size_t(rows)) throw std::runtime_error("CrossEntropyLoss: one target index per row of the logits");
    tensor<T> row_loss({rows});
    utils::CHECK_DF8(df8_cross_entropy_f32(logits.data(), pitch, nullptr, 0, idx.data(), rows, classes, row_loss.data(), fp8::stream()));
    const T mean = mean_of_rows(row_loss);
    check_indices();
    return mean;
}

template <typename T>
tensor<T> CrossEntropyLoss<T>::compute_gradient_pitched(const tensor<T>& logits, int classes, const tensor<int>& idx) {
    const auto& s = logits.shape();
    if (s.size() != 2 || classes <= 0 || s[1] < classes) throw std::runtime_error("CrossEntropyLoss::compute_gradient_pitched: logits must be [rows, pitch >= classes]");
    const int rows = s[0], pitch = s[1];
    if (idx.numel() != size_t(rows)) throw std::runtime_error("CrossEntropyLoss: one target index per row of the logits");
    tensor<T> grad({rows, classes});
    utils::CHECK_DF8(df8_cross_entropy_grad_f32(logits.data(), pitch, nullptr, 0, idx.data(), rows, classes, grad.data(), classes, fp8::stream()));
    utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));
    check_indices();
    return grad;
}

template class CrossEntropyLoss<float>;

}  // namespace dnn
