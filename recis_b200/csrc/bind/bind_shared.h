// Functions of one binding file that other binding files call directly (no trip through Python).
#pragma once
#include <torch/extension.h>
#include <tuple>

namespace rbx {

// bind_sparse.cpp
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> dedup_partition(
    const torch::Tensor& ids, int64_t world, c10::optional<torch::Tensor> unique_out, c10::optional<torch::Tensor> offsets_out,
    c10::optional<torch::Tensor> status, c10::optional<torch::Tensor> counts_out);
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> build_csr(const torch::Tensor& reverse);

}  // namespace rbx
