// Header-only C++ shim over the C ABI (venom_b200.h) with the method surface of the reference's host classes, so
// that a harness written against them switches libraries by changing a type name:
//
//   venom_b200::Format_sr_nm<T>   the methods of Format_sr_nm<T>, src/format/format_sr_nm.hpp:31-50 of UDC-GAC/venom
//                                 (init_from_dense, init_from_sparse, to_dense, get_hA_val / _metadata / _indices,
//                                 get_n / get_m / get_bm / get_vec_length / get_meta_vec_length,
//                                 transform_and_sync_device) plus Format<T>'s get_A_num_rows / _cols / _nnz;
//   venom_b200::Spatha<T, T2>     the methods of Spmm_CNN<T, T2> / Spatha<T, T2>, src/spmm/spmm.hpp:40-59 and
//                                 src/spmm/spatha_spmm.cpp:60-90: spmm(times, bm, bn, bk, wm, wn, wk, mm, mn, mk, nstage)
//                                 returning the mean kernel milliseconds of `times` launches, get_result(), get_sparse().
//
// Differences, all deliberate: errors throw std::runtime_error with the library's message (the reference exits or
// asserts); the compressor and decompressor run on the GPU; the tile arguments of spmm() are accepted and ignored
// (the library picks its own tiles); the random-instance generator Format_sr_nm::init is not part of the shim (the
// reference draws from the unseeded libc rand() stream) -- build instances with init_from_dense / init_from_sparse.
// T and T2 must be 16-bit floating point types (__half or any 2-byte stand-in); needs the CUDA runtime.
#ifndef VENOM_B200_SPATHA_HPP_
#define VENOM_B200_SPATHA_HPP_

#include <cuda_runtime_api.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "venom_b200.h"

namespace venom_b200 {

namespace detail {
inline void check(int rc, const char *what)
{
    if (rc != 0) throw std::runtime_error(std::string(what) + ": " + vnm_last_error_string());
}
inline void check_cuda(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
// Device buffer with the lifetime of a scope.
struct DeviceBuffer {
    void *p = nullptr;
    explicit DeviceBuffer(size_t bytes) { check_cuda(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc"); }
    DeviceBuffer(const void *host, size_t bytes) : DeviceBuffer(bytes) { check_cuda(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice), "cudaMemcpy"); }
    ~DeviceBuffer() { cudaFree(p); }
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
};
}  // namespace detail

template <class T>
class Format_sr_nm {
    static_assert(sizeof(T) == 2, "the V:N:M path is fp16: T must be a 2-byte type");

public:
    Format_sr_nm() = default;
    ~Format_sr_nm() { vnm_destroy(handle_); }
    Format_sr_nm(const Format_sr_nm &) = delete;
    Format_sr_nm &operator=(const Format_sr_nm &) = delete;

    // Compresses a dense (already pruned) row-major matrix with the given column-loc array on the GPU.
    // brow_ and mbrow_ are the reference's --block-size / --meta-block-size (the format is defined for 4 and 32).
    void init_from_dense(int nrow_, int ncol_, float density_, unsigned seed_, int n_, int m_, int brow_, int mbrow_, int bm_,
                         std::vector<T> &dense, std::vector<unsigned int> &columns)
    {
        set_shape(nrow_, ncol_, density_, seed_, n_, m_, brow_, mbrow_, bm_);
        if ((int64_t)dense.size() != (int64_t)nrow_ * ncol_) throw std::runtime_error("init_from_dense: dense must hold nrow * ncol elements");
        if ((int64_t)columns.size() != nc_) throw std::runtime_error("init_from_dense: column-loc array has the wrong size");
        hA_columns = columns;
        hA_values.assign((size_t)nv_, T());
        hA_metadata.assign((size_t)nm_, 0u);
        detail::DeviceBuffer d(dense.data(), dense.size() * 2), c(columns.data(), columns.size() * 4), v((size_t)nv_ * 2), md((size_t)nm_ * 4);
        detail::check(vnm_compress_f16(d.p, ncol_, nullptr, (const uint32_t *)c.p, nrow_, ncol_, bm_, n_, m_, v.p, (uint32_t *)md.p, nullptr, nullptr),
                      "vnm_compress_f16");
        detail::check_cuda(cudaMemcpy(hA_values.data(), v.p, (size_t)nv_ * 2, cudaMemcpyDeviceToHost), "cudaMemcpy");
        detail::check_cuda(cudaMemcpy(hA_metadata.data(), md.p, (size_t)nm_ * 4, cudaMemcpyDeviceToHost), "cudaMemcpy");
        initialized_ = true;
        drop_device();
    }

    // Adopts arrays that are already in the reference format.
    void init_from_sparse(int nrow_, int ncol_, float density_, unsigned seed_, int n_, int m_, int brow_, int mbrow_, int bm_,
                          std::vector<T> &values, std::vector<unsigned int> &columns_, std::vector<unsigned int> &metadata_)
    {
        set_shape(nrow_, ncol_, density_, seed_, n_, m_, brow_, mbrow_, bm_);
        if ((int64_t)values.size() != nv_ || (int64_t)columns_.size() != nc_ || (int64_t)metadata_.size() != nm_)
            throw std::runtime_error("init_from_sparse: array sizes do not match the format");
        hA_values = values;
        hA_columns = columns_;
        hA_metadata = metadata_;
        initialized_ = true;
        drop_device();
    }

    std::vector<T> &to_dense()
    {
        need_init();
        hA_dense.assign((size_t)A_num_rows * A_num_cols, T());
        detail::DeviceBuffer v(hA_values.data(), (size_t)nv_ * 2), md(hA_metadata.data(), (size_t)nm_ * 4), c(hA_columns.data(), (size_t)nc_ * 4),
            d(hA_dense.size() * 2);
        detail::check(vnm_decompress_f16(v.p, (const uint32_t *)md.p, (const uint32_t *)c.p, A_num_rows, A_num_cols, bm, n, m, d.p, A_num_cols, nullptr),
                      "vnm_decompress_f16");
        detail::check_cuda(cudaMemcpy(hA_dense.data(), d.p, hA_dense.size() * 2, cudaMemcpyDeviceToHost), "cudaMemcpy");
        return hA_dense;
    }

    // Uploads the arrays and re-packs them for the kernels (the reference packs metadata + indices into one allocation).
    void transform_and_sync_device()
    {
        need_init();
        drop_device();
        detail::DeviceBuffer v(hA_values.data(), (size_t)nv_ * 2), md(hA_metadata.data(), (size_t)nm_ * 4), c(hA_columns.data(), (size_t)nc_ * 4);
        detail::check(vnm_prepare(v.p, (const uint32_t *)md.p, (const uint32_t *)c.p, A_num_rows, A_num_cols, bm, n, m, &handle_, nullptr), "vnm_prepare");
        detail::check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }

    std::vector<unsigned int> &get_hA_metadata() { return hA_metadata; }
    std::vector<unsigned int> &get_hA_indices() { return hA_columns; }
    std::vector<T> &get_hA_val() { return hA_values; }
    int get_A_num_rows() const { return A_num_rows; }
    int get_A_num_cols() const { return A_num_cols; }
    int get_A_nnz() const { return (int)nv_; }
    int get_n() const { return n; }
    int get_m() const { return m; }
    int get_bm() const { return bm; }
    int get_vec_length() const { return brow; }
    int get_meta_vec_length() const { return mbrow; }
    vnm_handle_t device_handle()
    {
        if (!handle_) transform_and_sync_device();
        return handle_;
    }

private:
    void set_shape(int nrow_, int ncol_, float density_, unsigned seed_, int n_, int m_, int brow_, int mbrow_, int bm_)
    {
        if (brow_ != 4 || mbrow_ != 32) throw std::runtime_error("the storage format is defined for brow = 4 and mbrow = 32");
        int64_t ksp = 0;
        detail::check(vnm_sizes(nrow_, ncol_, bm_, n_, m_, &ksp, &nv_, &nm_, &nc_), "vnm_sizes");
        A_num_rows = nrow_; A_num_cols = ncol_; density = density_; seed = seed_;
        n = n_; m = m_; brow = brow_; mbrow = mbrow_; bm = bm_;
    }
    void need_init() const
    {
        if (!initialized_) throw std::runtime_error("Format_sr_nm: call init_from_dense or init_from_sparse first");
    }
    void drop_device()
    {
        vnm_destroy(handle_);
        handle_ = nullptr;
    }

    int A_num_rows = 0, A_num_cols = 0, n = 2, m = 0, brow = 4, mbrow = 32, bm = 0;
    float density = 0.f;
    unsigned seed = 0;
    int64_t nv_ = 0, nm_ = 0, nc_ = 0;
    bool initialized_ = false;
    std::vector<unsigned int> hA_metadata, hA_columns;
    std::vector<T> hA_values, hA_dense;
    vnm_handle_t handle_ = nullptr;
};

template <class T, class T2 = T>
class Spatha {
    static_assert(sizeof(T) == 2 && sizeof(T2) == 2, "only precision half is implemented");

public:
    // B_host: the dense operand [K, N] row-major on the host (the reference takes it from its Dataset).
    Spatha(Format_sr_nm<T> &f, const std::vector<T> &B_host, int B_num_cols)
        : fmt_(f), N_(B_num_cols), dB_(B_host.data(), B_host.size() * 2), dC_((size_t)f.get_A_num_rows() * B_num_cols * 2)
    {
        if ((int64_t)B_host.size() != (int64_t)f.get_A_num_cols() * B_num_cols) throw std::runtime_error("Spatha: B must hold K * N elements");
        fmt_.transform_and_sync_device();
        gflop_count = (float)f.get_A_num_rows() / 1e9f * B_num_cols * f.get_A_num_cols() * 2;
    }

    T *get_dB() { return (T *)dB_.p; }
    T2 *get_dC() { return (T2 *)dC_.p; }

    // One warm-up launch, then `times` launches timed with CUDA events; returns the mean milliseconds per launch and
    // leaves the result in get_result().  The tile arguments are the reference's and are ignored here.
    float spmm(int times, int bm_ = 0, int bn_ = 0, int bk_ = 0, int wm_ = 0, int wn_ = 0, int wk_ = 0, int mm_ = 0, int mn_ = 0, int mk_ = 0,
               int nstage_ = 0)
    {
        (void)bm_; (void)bn_; (void)bk_; (void)wm_; (void)wn_; (void)wk_; (void)mm_; (void)mn_; (void)mk_; (void)nstage_;
        vnm_handle_t h = fmt_.device_handle();
        const int M = fmt_.get_A_num_rows();
        auto launch = [&] { detail::check(vnm_spmm_f16(h, dB_.p, N_, N_, nullptr, dC_.p, N_, VNM_LAYOUT_MN, nullptr), "vnm_spmm_f16"); };
        launch();
        detail::check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        cudaEvent_t e0, e1;
        detail::check_cuda(cudaEventCreate(&e0), "cudaEventCreate");
        detail::check_cuda(cudaEventCreate(&e1), "cudaEventCreate");
        cudaEventRecord(e0);
        for (int i = 0; i < times; i++) launch();
        cudaEventRecord(e1);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        int status = 0;
        detail::check(vnm_device_status(h, &status, nullptr), "vnm_device_status");
        result_.resize((size_t)M * N_);
        detail::check_cuda(cudaMemcpy(result_.data(), dC_.p, result_.size() * 2, cudaMemcpyDeviceToHost), "cudaMemcpy");
        return times > 0 ? ms / times : 0.f;
    }

    std::vector<T2> &get_result() { return result_; }
    std::vector<T> &get_sparse() { throw std::runtime_error("Operation not supported yet"); }
    float get_gflop_count() const { return gflop_count; }

private:
    Format_sr_nm<T> &fmt_;
    int N_;
    detail::DeviceBuffer dB_, dC_;
    std::vector<T2> result_;
    float gflop_count = 0.f;
};

}  // namespace venom_b200

#endif  // VENOM_B200_SPATHA_HPP_
