// A C++ consumer of the additive libreCu* entry points (memset, directional copies, pinned host memory,
// cross-stream event waits, event queries, the shard partitioner and the partitioned copy), written the way
// the reference's own test programs use its API (tests/memcopy/main.cpp:1-75 there): include <librecuda.h>,
// link the `driverapi` library, check every status.  Verifies results against host computations and prints
// "additive API ok".  Needs one GPU.
#include <lcb200_kernels.h>
#include <librecuda.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#define CHECK(expr)                                                                                   \
    do {                                                                                              \
        libreCudaStatus_t status_ = (expr);                                                           \
        if (status_ != LIBRECUDA_SUCCESS) {                                                           \
            const char *name_ = nullptr;                                                              \
            libreCuGetErrorString(status_, &name_);                                                   \
            std::fprintf(stderr, "%s:%d: %s -> %s\n", __FILE__, __LINE__, #expr, name_ ? name_ : "?"); \
            std::exit(1);                                                                             \
        }                                                                                             \
    } while (0)

#define EXPECT(cond)                                                               \
    do {                                                                           \
        if (!(cond)) {                                                             \
            std::fprintf(stderr, "%s:%d: expected %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                          \
        }                                                                          \
    } while (0)

int main() {
    CHECK(libreCuInit(0));
    LibreCUdevice device{};
    CHECK(libreCuDeviceGet(&device, 0));
    LibreCUcontext ctx{};
    CHECK(libreCuCtxCreate_v2(&ctx, CU_CTX_SCHED_YIELD, device));
    LibreCUstream a{}, b{};
    CHECK(libreCuStreamCreate(&a, 0));
    CHECK(libreCuStreamCreate(&b, 0));

    const size_t n = (size_t)5 << 20;  // 5 MiB + odd tails below
    uint8_t *dev0 = nullptr, *dev1 = nullptr;
    CHECK(libreCuMemAlloc(reinterpret_cast<void **>(&dev0), n + 64));
    CHECK(libreCuMemAlloc(reinterpret_cast<void **>(&dev1), n + 64));
    uint8_t *pinned = nullptr;
    CHECK(libreCuMemAllocHost(reinterpret_cast<void **>(&pinned), n + 64));
    std::vector<uint8_t> pageable(n + 64), expect(n + 64);

    // memset of three widths, ragged counts and offsets, then a directional copy back
    CHECK(libreCuMemsetD8(dev0, 0xA5, n + 64, a));
    CHECK(libreCuMemsetD32(dev0 + 4, 0x40490FDBu, (n - 8) / 4, a));
    CHECK(libreCuMemsetD16(dev0 + n - 2, 0xBEEF, 7, a));
    CHECK(libreCuMemsetD8(dev0 + 1, 0x11, 2, a));
    CHECK(libreCuMemcpyDtoH(pageable.data(), dev0, n + 64, a));
    CHECK(libreCuStreamCommence(a));
    CHECK(libreCuStreamAwait(a));
    std::memset(expect.data(), 0xA5, n + 64);
    for (size_t i = 0; i < (n - 8) / 4; ++i) {
        const uint32_t v = 0x40490FDBu;
        std::memcpy(expect.data() + 4 + 4 * i, &v, 4);
    }
    for (size_t i = 0; i < 7; ++i) {
        const uint16_t v = 0xBEEF;
        std::memcpy(expect.data() + n - 2 + 2 * i, &v, 2);
    }
    expect[1] = expect[2] = 0x11;
    EXPECT(std::memcmp(pageable.data(), expect.data(), n + 64) == 0);

    // direction checks: a host pointer where a device pointer belongs is refused
    EXPECT(libreCuMemcpyHtoD(pageable.data(), pinned, 16, a) == LIBRECUDA_ERROR_INVALID_VALUE);
    EXPECT(libreCuMemcpyDtoD(dev0, pinned, 16, a) == LIBRECUDA_ERROR_INVALID_VALUE);
    EXPECT(libreCuMemsetD32(dev0 + 2, 1, 4, a) == LIBRECUDA_ERROR_INVALID_VALUE);  // misaligned for its width

    // stream b consumes what stream a produces: HtoD on a, event, wait on b, misaligned DtoD + DtoH on b
    for (size_t i = 0; i < n + 64; ++i) pinned[i] = (uint8_t)((i * 2654435761u) >> 24);
    LibreCUEvent produced{}, start{}, stop{};
    CHECK(libreCuEventCreate(&produced, 0));
    CHECK(libreCuEventCreate(&start, 0));
    CHECK(libreCuEventCreate(&stop, 0));
    EXPECT(libreCuEventQuery(produced) == LIBRECUDA_ERROR_INVALID_VALUE);  // never recorded
    CHECK(libreCuMemcpyHtoD(dev0, pinned, n + 64, a));
    CHECK(libreCuEventRecord(produced, a));
    EXPECT(libreCuEventQuery(produced) == LIBRECUDA_ERROR_NOT_READY);      // recorded, not commenced
    CHECK(libreCuStreamWaitEvent(b, produced));
    CHECK(libreCuEventRecord(start, b));
    CHECK(libreCuMemcpyDtoD(dev1 + 3, dev0 + 1, n, b));
    CHECK(libreCuEventRecord(stop, b));
    CHECK(libreCuMemcpyDtoH(pageable.data(), dev1 + 3, n, b));
    EXPECT(libreCuStreamCommence(b) == LIBRECUDA_ERROR_NOT_READY);  // the producer has not been submitted yet
    CHECK(libreCuStreamCommence(a));
    CHECK(libreCuStreamCommence(b));
    CHECK(libreCuStreamAwait(b));
    CHECK(libreCuStreamAwait(a));
    EXPECT(std::memcmp(pageable.data(), pinned + 1, n) == 0);
    CHECK(libreCuEventQuery(produced));
    float ms = -1.f;
    CHECK(libreCuEventElapsedTime(&ms, start, stop));
    EXPECT(ms > 0.f);
    uint64_t t_produced = 0, t_start = 0;
    CHECK(libreCuEventGetTimestamp(&t_produced, produced));
    CHECK(libreCuEventGetTimestamp(&t_start, start));
    EXPECT(t_start >= t_produced);  // the wait held

    // partitioner: 2 MiB-aligned shards that cover the range exactly; partitioned copy onto this one GPU
    size_t off[4] = {};
    CHECK(libreCuPartitionPlan(n + 5, 3, 0, off));
    EXPECT(off[0] == 0 && off[3] == n + 5);
    EXPECT(off[1] % ((size_t)2 << 20) == 0 && off[2] % ((size_t)2 << 20) == 0);
    EXPECT(off[0] <= off[1] && off[1] <= off[2] && off[2] <= off[3]);
    CHECK(libreCuMemsetD8(dev1, 0, n + 64, a));
    void *dsts[3] = {dev1 + off[0], dev1 + off[1], dev1 + off[2]};
    LibreCUstream streams[3] = {a, a, a};
    CHECK(libreCuMemcpyPartitioned(dsts, dev0, n + 5, 3, 0, streams));
    CHECK(libreCuMemcpyDtoH(pageable.data(), dev1, n + 64, a));
    CHECK(libreCuStreamCommence(a));
    CHECK(libreCuStreamAwait(a));
    EXPECT(std::memcmp(pageable.data(), pinned, n + 5) == 0);
    EXPECT(pageable[n + 5] == 0 && pageable[n + 63] == 0);  // nothing written past the range

    int can = -1;
    CHECK(libreCuDeviceCanAccessPeer(&can, device, device));
    EXPECT(can == 1);
    void *native = nullptr;
    CHECK(libreCuStreamGetNativeHandle(&native, a));
    EXPECT(native != nullptr);

    // the kernel layer underneath, on the stream's native handle: the plan query names what will be launched, a
    // copy whose source nothing in flight writes may load ahead of the stream wait, and a bounded wait that runs
    // out shows up as the status of the next Await (once), not as a hang or a CUDA error
    char plan[200] = {};
    EXPECT(lcb_copy_d2d_describe(dev1, dev0, n, LCB_COPY_AUTO | LCB_COPY_SRC_STABLE, 0, plan, sizeof(plan)) == 0);
    EXPECT(std::strstr(plan, "copy_vec_kernel<-1,") == plan && std::strstr(plan, "loads before the stream wait") != nullptr);
    EXPECT(lcb_copy_d2d_describe(dev1, dev0 + 1, n, LCB_COPY_TMA, 0, plan, sizeof(plan)) == 1);  // bulk path needs congruent pointers
    CHECK(libreCuMemsetD8(dev1, 0, n + 64, a));
    CHECK(libreCuStreamCommence(a));
    CHECK(libreCuStreamAwait(a));
    for (int rep = 0; rep < 4; ++rep)
        EXPECT(lcb_copy_d2d_ex(dev1 + 5, dev0 + 2, n, LCB_COPY_AUTO | LCB_COPY_SRC_STABLE, 0, native) == 0);
    CHECK(libreCuMemcpyDtoH(pageable.data(), dev1 + 5, n, a));
    CHECK(libreCuStreamCommence(a));
    CHECK(libreCuStreamAwait(a));
    EXPECT(std::memcmp(pageable.data(), pinned + 2, n) == 0);
    EXPECT(lcb_flag_wait(dev1, 1, 0, native) == 1);                 // a wait without a limit is refused
    EXPECT(lcb_flag_wait(dev1, 0x7fffffffu, 50, native) == 0);      // nobody posts this value: gives up after 50 ms
    EXPECT(libreCuStreamAwait(a) == LIBRECUDA_ERROR_UNKNOWN);       // reported once ...
    CHECK(libreCuStreamAwait(a));                                   // ... then clear, and the stream still works
    EXPECT(lcb_flag_post(dev1, 7, native) == 0);
    EXPECT(lcb_flag_wait(dev1, 7, 1000, native) == 0);
    CHECK(libreCuStreamAwait(a));

    CHECK(libreCuEventDestroy(produced));
    CHECK(libreCuEventDestroy(start));
    CHECK(libreCuEventDestroy(stop));
    CHECK(libreCuMemFreeHost(pinned));
    CHECK(libreCuMemFree(dev0));
    CHECK(libreCuMemFree(dev1));
    CHECK(libreCuStreamDestroy(a));
    CHECK(libreCuStreamDestroy(b));
    CHECK(libreCuCtxDestroy(ctx));
    std::printf("additive API ok\n");
    return 0;
}
