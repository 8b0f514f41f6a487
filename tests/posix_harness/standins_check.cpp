// Drives the POSIX stand-ins of oracle/posix/ through the reference's own headers (safetensors.h, image_io.h, windows.h
// uses) and prints what it read, one fact per line, for tests/test_posix_standins.py to compare with what Python wrote.
#include <windows.h>

#include <cstdio>
#include <stdexcept>
#include <string>

#include "image_io.h"
#include "safetensors.h"

static const char* dtype_name(DType d) {
    switch (d) {
        case DType::BF16: return "BF16";
        case DType::F16: return "F16";
        case DType::F32: return "F32";
        case DType::I64: return "I64";
        default: return "Other";
    }
}

int main(int argc, char** argv) {
    if (argc < 3) return 2;
    const std::string mode = argv[1], path = argv[2];
    try {
        if (mode == "tensors") {
            SafeTensors st(path);
            for (const auto& kv : st.all()) {
                printf("tensor %s %s", kv.first.c_str(), dtype_name(kv.second.dtype));
                for (auto d : kv.second.shape) printf(" %lld", (long long)d);
                printf(" | bytes %zu |", kv.second.bytes);
                const long long n = kv.second.numel();
                try {
                    for (long long i = 0; i < n && i < 4; i++) printf(" %.9g", st_elem_f32(kv.second, i));
                    if (n > 0) printf(" .. %.9g", st_elem_f32(kv.second, n - 1));
                } catch (const std::exception& e) { printf(" no float view: %s", e.what()); }
                printf("\n");
            }
            try { st.get("no.such.tensor"); } catch (const std::exception& e) { printf("missing: %s\n", e.what()); }
        } else if (mode == "image") {
            int w = 0, h = 0;
            std::vector<uint8_t> rgb;
            std::string err;
            if (!load_image_rgb(path, w, h, rgb, err)) { printf("image error: %s\n", err.c_str()); return 0; }
            unsigned long long sum = 0;
            for (size_t i = 0; i < rgb.size(); i++) sum += (unsigned long long)rgb[i] * (i % 251 + 1);
            printf("image %d %d %zu %llu first %d %d %d last %d %d %d\n", w, h, rgb.size(), sum, rgb[0], rgb[1], rgb[2], rgb[rgb.size() - 3],
                   rgb[rgb.size() - 2], rgb[rgb.size() - 1]);
        } else if (mode == "files") {
            printf("exists %d\n", GetFileAttributesA(path.c_str()) != INVALID_FILE_ATTRIBUTES);
            printf("icmp %d\n", _stricmp("Models\\Anima.SafeTensors", "models\\anima.safetensors"));
            printf("deleted %d\n", DeleteFileA(path.c_str()));
            printf("exists %d\n", GetFileAttributesA(path.c_str()) != INVALID_FILE_ATTRIBUTES);
        }
    } catch (const std::exception& e) {
        printf("exception: %s\n", e.what());
    }
    return 0;
}
