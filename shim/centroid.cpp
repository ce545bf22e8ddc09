// tensor::centroid::CentroidAccumulator and CentroidMerge (include/tensor/centroid/centroid_accumulator.hpp:24-53,
// centroid_merge.hpp:12-19; src/centroid/centroid_accumulator.cpp:16-168, centroid_merge.cpp:12-31) on the
// library: accumulation and the k-means merge run on the GPU, the file layouts are the reference's.
//
// The class layout is fixed by the reference's header (host vector + scalar), so the running sums live in a
// device buffer registered per object and are copied into acc_ / acc_weight_ when a snapshot is written.
#include <tensor/centroid/centroid_accumulator.hpp>
#include <tensor/centroid/centroid_merge.hpp>

#include <filesystem>
#include <fstream>
#include <iostream>
#include <map>
#include <stdexcept>

#include "shim_ctx.hpp"

namespace fs = std::filesystem;

namespace tensor::centroid {

namespace {
struct DeviceSums { float* acc = nullptr; float* weight = nullptr; };
std::map<const CentroidAccumulator*, DeviceSums>& registry() {
    static std::map<const CentroidAccumulator*, DeviceSums> r;
    return r;
}
}  // namespace

CentroidAccumulator::CentroidAccumulator(int D, const std::string& dir) : D_(D), dir_(dir), acc_(D, 0.f) {
    fs::create_directories(dir);
}

// acc += sum_t h_t * ||g_t||, weight += sum_t ||g_t||.  As in the reference (centroid_accumulator.cpp:45-48)
// both tensors are read through their BF16 pointer whatever their dtype tag says.
void CentroidAccumulator::accumulate(const backend::cuda::Tensor& hidden, const backend::cuda::Tensor& grad_signal,
                                     const backend::cuda::Device& dev) {
    const int BT = int(hidden.shape()[0]), D = int(hidden.shape()[1]);
    if (D != D_) return;
    DeviceSums& s = registry()[this];
    if (!s.acc) {
        CUDA_CHECK(cudaMalloc(&s.acc, sizeof(float) * (std::size_t(D) + 64)));
        CUDA_CHECK(cudaMemsetAsync(s.acc, 0, sizeof(float) * (std::size_t(D) + 64), dev.stream()));
        s.weight = s.acc + (std::size_t(D) + 63) / 64 * 64;
    }
    ta_shim::check(ta_centroid_accumulate(ta_shim::ctx(), TA_CENTROID_INTENDED, hidden.bf16(), grad_signal.bf16(), BT, D, s.acc,
                                          s.weight, ta_shim::as_stream(dev.stream())),
                   "CentroidAccumulator::accumulate");
    samples_ += std::size_t(BT);
}

void CentroidAccumulator::write_snapshot(std::size_t step) {
    auto it = registry().find(this);
    if (it != registry().end() && it->second.acc) {
        CUDA_CHECK(cudaDeviceSynchronize());
        CUDA_CHECK(cudaMemcpy(acc_.data(), it->second.acc, sizeof(float) * std::size_t(D_), cudaMemcpyDeviceToHost));
        CUDA_CHECK(cudaMemcpy(&acc_weight_, it->second.weight, sizeof(float), cudaMemcpyDeviceToHost));
    }
    if (acc_weight_ == 0.f) return;
    std::vector<float> centroid(static_cast<std::size_t>(D_));
    for (int d = 0; d < D_; d++) centroid[d] = acc_[d] / acc_weight_;
    const std::string path = dir_ + "/step-" + std::to_string(step) + ".centroid";
    std::ofstream f(path, std::ios::binary);
    f.write(reinterpret_cast<const char*>(&D_), sizeof(int));
    f.write(reinterpret_cast<const char*>(centroid.data()), std::streamsize(D_) * sizeof(float));
    f.write(reinterpret_cast<const char*>(&acc_weight_), sizeof(float));
    f.close();
    snapshots_.push_back(centroid);
    std::cerr << "[centroid] snapshot → " << path << " (weight=" << acc_weight_ << ")\n";
}

// k-means over the in-memory snapshots, else over the directory's files in iteration order
// (centroid_accumulator.cpp:93-168), clustered by ta_kmeans_merge on the GPU: bit-identical centres.
void CentroidAccumulator::merge_and_write(int k, const std::string& out_path) {
    if (snapshots_.empty()) {
        int n = 0, passes = 0;
        const int rc = ta_centroid_merge_dir(ta_shim::ctx(), dir_.c_str(), out_path.c_str(), k, &n, &passes);
        if (rc == TA_OK && n == 0) { std::cerr << "[centroid] no snapshots to merge\n"; return; }
        ta_shim::check(rc, "CentroidAccumulator::merge_and_write");
        std::cerr << "[centroid] merged " << n << " snapshots → " << out_path << "\n";
        return;
    }
    const int N = int(snapshots_.size()), D = D_, kk = std::min(k, N);
    std::vector<float> flat(std::size_t(N) * D);
    for (int i = 0; i < N; i++) std::copy(snapshots_[i].begin(), snapshots_[i].end(), flat.begin() + std::size_t(i) * D);
    float *d_vec = nullptr, *d_cen = nullptr; int* d_asg = nullptr;
    CUDA_CHECK(cudaMalloc(&d_vec, flat.size() * sizeof(float)));
    CUDA_CHECK(cudaMalloc(&d_cen, std::size_t(kk) * D * sizeof(float)));
    CUDA_CHECK(cudaMalloc(&d_asg, std::size_t(N) * sizeof(int)));
    CUDA_CHECK(cudaMemcpy(d_vec, flat.data(), flat.size() * sizeof(float), cudaMemcpyHostToDevice));
    int k_out = 0, passes = 0;
    const int rc = ta_kmeans_merge(ta_shim::ctx(), d_vec, N, D, k, 50, d_cen, d_asg, &k_out, &passes, nullptr);
    std::vector<float> centers(std::size_t(kk) * D);
    if (rc == TA_OK) cudaMemcpy(centers.data(), d_cen, centers.size() * sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(d_vec); cudaFree(d_cen); cudaFree(d_asg);
    ta_shim::check(rc, "CentroidAccumulator::merge_and_write");
    std::ofstream f(out_path, std::ios::binary);
    f.write(reinterpret_cast<const char*>(&k_out), sizeof(int));
    f.write(reinterpret_cast<const char*>(&D), sizeof(int));
    f.write(reinterpret_cast<const char*>(centers.data()), std::streamsize(k_out) * D * sizeof(float));
    std::cerr << "[centroid] merged " << N << " snapshots → " << out_path << "\n";
}

void CentroidMerge::run(const std::string& snapshot_dir, const std::string& out_path, int k) {
    int D = 0;
    for (const auto& e : fs::directory_iterator(snapshot_dir))
        if (e.path().extension() == ".centroid") {
            std::ifstream f(e.path(), std::ios::binary);
            f.read(reinterpret_cast<char*>(&D), sizeof(int));
            break;
        }
    if (D == 0) throw std::runtime_error("No .centroid files in " + snapshot_dir);
    CentroidAccumulator acc(D, snapshot_dir);
    acc.merge_and_write(k, out_path);
}

}  // namespace tensor::centroid
