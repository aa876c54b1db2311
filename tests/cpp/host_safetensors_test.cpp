// vai::SafetensorsParser / Checkpoint / loadTensor / concat / slice (vai_b200/host/safetensors.h).
//   host_safetensors_test <file>            prints one line per tensor: name, dtype, shape, byte
//                                           size and FNV-1a sums of the tensor converted to
//                                           F32 / F16 / BF16 on the host (compared by the caller)
//   host_safetensors_test <file> --gpu      also loads every tensor to the device in each dtype,
//                                           reads it back and compares it with the host conversion;
//                                           then concat and slice of the first 2-D tensor
#include <cstdio>

#include "../../vai_b200/host/safetensors.h"

using namespace vai;

static uint64_t fnv(const void* p, size_t n)
{
    uint64_t h = 1469598103934665603ull;
    const uint8_t* b = static_cast<const uint8_t*>(p);
    for (size_t i = 0; i < n; ++i) h = (h ^ b[i]) * 1099511628211ull;
    return h;
}

static std::vector<uint8_t> hostConvert(const SafetensorRef& ref, Dtype to)
{
    const Dtype from = detail::dtypeOfFile(ref.getDataType());
    const size_t count = ref.byteSize() / bytesPerElement(from);
    std::vector<uint8_t> out(count * bytesPerElement(to));
    detail::convertStored(ref.data(), from, out.data(), to, count);
    return out;
}

int main(int argc, char** argv)
{
    if (argc < 2) return 2;
    const bool gpu = argc > 2 && std::string(argv[2]) == "--gpu";
    int fails = 0;
    try {
        SafetensorsParser parser(argv[1]);
        std::vector<std::string> names = parser.getTensorNames();
        std::sort(names.begin(), names.end());
        const Dtype all[3] = {Dtype::Fp32, Dtype::Fp16, Dtype::Bf16};
        std::string first2d;
        for (const std::string& name : names) {
            SafetensorRef ref = parser[name];
            std::printf("%s %s", name.c_str(), ref.getDataType().c_str());
            for (uint32_t s : ref.getShape()) std::printf(" %u", s);
            std::printf(" | %zu", ref.byteSize());
            for (Dtype to : all) {
                std::vector<uint8_t> h = hostConvert(ref, to);
                std::printf(" %016llx", (unsigned long long)fnv(h.data(), h.size()));
                if (gpu) {
                    Tensor t = loadTensor(ref, to);
                    std::vector<uint8_t> back(t.numBytes());
                    t.download(back.data());
                    vaicu_device_synchronize(deviceHandle());
                    if (back != h || t.shape() != ref.getShape()) { std::printf(" DEVICE-MISMATCH"); ++fails; }
                }
            }
            std::printf("\n");
            if (first2d.empty() && ref.getShape().size() == 2 && ref.getShape()[0] >= 2) first2d = name;
        }
        if (gpu && !first2d.empty()) {
            SafetensorRef ref = parser[first2d];
            const std::vector<uint32_t> shape = ref.getShape();
            std::vector<uint8_t> h = hostConvert(ref, Dtype::Bf16);
            Tensor both = concat({ref, ref}, Dtype::Bf16);
            std::vector<uint8_t> back(both.numBytes());
            both.download(back.data());
            vaicu_device_synchronize(deviceHandle());
            const bool okConcat = both.shape()[0] == 2 * shape[0] && back.size() == 2 * h.size() &&
                                  std::equal(h.begin(), h.end(), back.begin()) && std::equal(h.begin(), h.end(), back.begin() + h.size());
            Tensor part = slice(ref, 1, shape[0], Dtype::Bf16);
            std::vector<uint8_t> rows(part.numBytes());
            part.download(rows.data());
            vaicu_device_synchronize(deviceHandle());
            const size_t rowBytes = h.size() / shape[0];
            const bool okSlice = part.shape()[0] == shape[0] - 1 && std::equal(rows.begin(), rows.end(), h.begin() + rowBytes);
            std::printf("concat %s slice %s\n", okConcat ? "ok" : "MISMATCH", okSlice ? "ok" : "MISMATCH");
            fails += !okConcat + !okSlice;
        }
        bool threw = false;
        try { parser.getShape("no.such.tensor"); } catch (const std::out_of_range&) { threw = true; }
        if (!threw) { std::printf("missing key did not throw\n"); ++fails; }
    } catch (const std::exception& e) {
        std::printf("error: %s\n", e.what());
        return 3;
    }
    return fails ? 1 : 0;
}
