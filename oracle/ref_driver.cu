// Thin extern "C" driver around the reference's own Format_sr_nm<__half> class.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no reference code: it includes the reference headers
// by path and is compiled together with the reference's src/format/format.cpp and
// src/format/format_sr_nm.cpp, where they lie in the read-only reference checkout, by
// oracle/build_oracle.py.  The resulting oracle/_ref/libvnm_ref.so is used to pin the C restatement in
// vnm_oracle.c and to generate the golden vectors; it is never loaded by the product path.
#include "format/format_sr_nm.hpp"
#include <cstring>
#include <cstdint>
#include <cstdio>
#include <unistd.h>
#include <fcntl.h>

namespace {
// init_from_dense prints two progress lines to stdout (format_sr_nm.cpp:138,147); silence them.
struct QuietStdout {
    int saved;
    QuietStdout() { fflush(stdout); saved = dup(1); int n = open("/dev/null", O_WRONLY); dup2(n, 1); close(n); }
    ~QuietStdout() { std::cout.flush(); fflush(stdout); dup2(saved, 1); close(saved); }
};
}

extern "C" {

// Format_sr_nm<__half>::init_from_dense -> to_sparse_sr_nm (format_sr_nm.cpp:108-149, 419-543).
int ref_compress_f16(const uint16_t* dense, const uint32_t* columns, int M, int K, int V, int m,
                     uint16_t* values, uint32_t* meta, long values_elems, long meta_words, long col_words)
{
    std::vector<__half> d((size_t)M * K);
    std::memcpy(d.data(), dense, d.size() * 2);
    std::vector<uint> c(columns, columns + col_words);
    Format_sr_nm<__half> f;
    {
        QuietStdout q;
        f.init_from_dense(M, K, 2.0f / m, 0, 2, m, 4, 32, V, d, c);
    }
    if ((long)f.get_hA_val().size() != values_elems || (long)f.get_hA_metadata().size() != meta_words) return 1;
    std::memcpy(values, f.get_hA_val().data(), values_elems * 2);
    std::memcpy(meta, f.get_hA_metadata().data(), meta_words * 4);
    return 0;
}

// Format_sr_nm<__half>::init_from_sparse + to_dense (format_sr_nm.cpp:77-106, 327-417).
int ref_to_dense_f16(const uint16_t* values, const uint32_t* meta, const uint32_t* columns,
                     int M, int K, int V, int m, long values_elems, long meta_words, long col_words,
                     uint16_t* dense)
{
    std::vector<__half> v(values_elems);
    std::memcpy(v.data(), values, values_elems * 2);
    std::vector<uint> c(columns, columns + col_words);
    std::vector<uint> md(meta, meta + meta_words);
    Format_sr_nm<__half> f;
    f.init_from_sparse(M, K, 2.0f / m, 0, 2, m, 4, 32, V, v, c, md);
    std::vector<__half>& out = f.to_dense();
    if (out.size() != (size_t)M * K) return 1;
    std::memcpy(dense, out.data(), out.size() * 2);
    return 0;
}

// Format_sr_nm<__half>::init (format_sr_nm.cpp:31-75): the reference's own random instance
// (libc rand() stream; values rand()%9-4).  srand(seed) is called here so runs are repeatable.
int ref_random_init_f16(int M, int K, int V, int m, unsigned seed,
                        uint16_t* values, uint32_t* meta, uint32_t* columns,
                        long values_elems, long meta_words, long col_words)
{
    std::srand(seed);
    Format_sr_nm<__half> f;
    f.init(M, K, 2, 2.0f / m, seed, false, m, 4, 32, V);
    if ((long)f.get_hA_val().size() != values_elems || (long)f.get_hA_metadata().size() != meta_words ||
        (long)f.get_hA_indices().size() != col_words) return 1;
    std::memcpy(values, f.get_hA_val().data(), values_elems * 2);
    std::memcpy(meta, f.get_hA_metadata().data(), meta_words * 4);
    std::memcpy(columns, f.get_hA_indices().data(), col_words * 4);
    return 0;
}

}
