// The C++ mirror of the cache2 page-table manager (include/sg_gpu.hpp, PageCache) over the C ABI: a second
// sequence with the same first two pages of tokens shares their physical pages.  Host only, no GPU.
#include <cstdio>
#include <numeric>

#include "sg_gpu.hpp"

int main()
{
    try {
        sg_gpu::PageCache cache(8, 16);
        std::vector<int32_t> a(40);
        std::iota(a.begin(), a.end(), 100);
        if (cache.lookup(a) != 0) return 1;
        auto sa = cache.acquire(a, 64);
        if (sa.reused_tokens != 0 || sa.table.size() != 4) return 2;
        cache.commit(sa, a);
        if (cache.lookup(a) != 32) return 3;
        std::vector<int32_t> b(a.begin(), a.begin() + 36);
        b.push_back(7);
        auto sb = cache.acquire(b);
        if (sb.reused_tokens != 32 || sb.table[0] != sa.table[0] || sb.table[1] != sa.table[1] || sb.table[2] == sa.table[2]) return 4;
        cache.release(sa);
        cache.release(sb);
        const auto st = cache.stats();
        if (st.live_sequences != 0 || st.hits != 1 || st.misses != 1) return 5;
        bool threw = false;
        try {
            sg_gpu::PageCache bad(4, 24);  // not a power of two
        } catch (const sg_gpu::Validation&) {
            threw = true;
        }
        if (!threw) return 6;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "unexpected: %s\n", e.what());
        return 9;
    }
    std::puts("page cache ok");
    return 0;
}
