// Host-only exercise of lcu::CopyPool for the sanitizer builds: many copies of odd sizes and alignments,
// pool creation and destruction, results compared with plain memcpy.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "copy_pool.h"

int main() {
    const size_t kMax = (size_t)3 << 20;
    std::vector<unsigned char> src(kMax + 64), dst(kMax + 64), want(kMax + 64);
    for (size_t i = 0; i < src.size(); ++i) src[i] = (unsigned char)(i * 2654435761u >> 13);
    const size_t sizes[] = {0, 1, 4095, 4096, 4097, (1u << 20) - 1, 1u << 20, (1u << 20) + 1, (2u << 20) + 12345, kMax};
    for (int workers : {1, 3, 8}) {
        lcu::CopyPool pool(workers);
        for (int round = 0; round < 2; ++round)
            for (size_t n : sizes)
                for (size_t off : {(size_t)0, (size_t)63}) {
                    std::fill(dst.begin(), dst.end(), 0xAA);
                    std::fill(want.begin(), want.end(), 0xAA);
                    pool.copy(dst.data() + off, src.data() + 7, n, /*streaming=*/(round & 1) != 0);
                    std::memcpy(want.data() + off, src.data() + 7, n);
                    if (dst != want) {
                        std::printf("mismatch: workers %d size %zu off %zu\n", workers, n, off);
                        return 1;
                    }
                }
    }
    std::printf("copy pool ok\n");
    return 0;
}
