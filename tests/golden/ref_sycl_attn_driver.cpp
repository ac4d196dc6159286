// ref_sycl_attn_driver.cpp — fixture generator (TEST INFRASTRUCTURE, not product).
//
// Runs the reference's OWN decode attention — nova::syclk::attn_decode
// (src/kernel/sycl/attn.cpp:41-161), the structural twin of fa_split_kernel +
// fa_combine_kernel (src/kernel/attn.cu:90-191) — on the CPU through the
// reference's thread-per-work-item SYCL stand-in (tests/host_sycl/sycl/sycl.hpp),
// on inputs read from a file, and writes its output.  Built and driven by
// tests/golden/make_golden.py from the reference tree where it lies; the
// reference sources are only #included, never copied.
//
// usage: driver <in.bin> <out.bin>
//   in : int32 n_keys, then q[NH*HD], kc[n_keys*NKV*HD], vc[n_keys*NKV*HD] as fp32
//   out: o[NH*HD] fp32
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "attn.cpp"   // found on the reference's src/kernel/sycl include path

int main(int argc, char** argv) {
    if (argc != 3) return 2;
    std::FILE* f = std::fopen(argv[1], "rb");
    if (!f) return 3;
    int n_keys = 0;
    if (std::fread(&n_keys, 4, 1, f) != 1 || n_keys <= 0) return 4;
    const int NH = nova::syclk::kNH, NKV = nova::syclk::kNKV, HD = nova::syclk::kHD;
    std::vector<float> q((size_t)NH * HD), kc((size_t)n_keys * NKV * HD), vc(kc.size()), o(q.size());
    if (std::fread(q.data(), 4, q.size(), f) != q.size()) return 5;
    if (std::fread(kc.data(), 4, kc.size(), f) != kc.size()) return 5;
    if (std::fread(vc.data(), 4, vc.size(), f) != vc.size()) return 5;
    std::fclose(f);
    std::vector<float> scratch((size_t)nova::syclk::attn_decode_scratch_floats());
    sycl::queue queue;
    nova::syclk::attn_decode(q.data(), kc.data(), vc.data(), o.data(), n_keys - 1, scratch.data(), queue);
    queue.wait();
    f = std::fopen(argv[2], "wb");
    if (!f) return 6;
    std::fwrite(o.data(), 4, o.size(), f);
    std::fclose(f);
    std::printf("NH=%d NKV=%d HD=%d n_keys=%d\n", NH, NKV, HD, n_keys);
    return 0;
}
