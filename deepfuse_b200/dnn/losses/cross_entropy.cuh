// CrossEntropyLoss<T>: upstream's class (dnn/losses/cross_entropy.cuh:8-20) on df8_cross_entropy_f32.
//
// Same four entry points and the same arithmetic (softmax with the row maximum taken out, 1e-7 added to the sum of
// exponentials, mean over the rows accumulated on the host in row order as upstream does, cross_entropy.cu:155-168).
// Differences: rows = every leading dimension (upstream takes shape()[0] x shape()[1], which is wrong for [B,T,V]
// logits); class-index targets are used as they are (upstream first builds a one-hot matrix the size of the logits,
// utils/common.cuh:123); compute_pitched / compute_gradient_pitched read logits whose rows are `pitch` floats apart
// (Gpt2::forward_logits_pitched).  An index outside [0, classes) throws.
#pragma once

#include "dnn/losses/loss.cuh"

namespace dnn {

template <typename T>
class CrossEntropyLoss : public Loss<T> {
public:
    CrossEntropyLoss() = default;

    T compute(const tensor<T>& predictions, const tensor<T>& targets) override;
    tensor<T> compute_gradient(const tensor<T>& predictions, const tensor<T>& targets) override;
    // class-index targets: one index per row of the logits
    T compute(const tensor<T>& predictions, const tensor<int>& target_indices);
    tensor<T> compute_gradient(const tensor<T>& predictions, const tensor<int>& target_indices);
    // logits [rows, pitch] of which the first `classes` columns count; the gradient comes back dense [rows, classes]
    T compute_pitched(const tensor<T>& predictions, int classes, const tensor<int>& target_indices);
    tensor<T> compute_gradient_pitched(const tensor<T>& predictions, int classes, const tensor<int>& target_indices);

private:
    T mean_of_rows(const tensor<T>& row_loss) const;
};

}  // namespace dnn
