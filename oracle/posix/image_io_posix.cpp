// load_image_rgb (interface: engine/src/image_io.h:9) without the Windows Imaging Component, for the Linux build of the
// reference's engine that the tests drive as the checker. The reference decodes any format the system codecs know
// (engine/src/image_io.cpp:20-80); a headless test session needs only formats that need no codec, so this reads binary
// PPM (P6, 8 bits per channel) and uncompressed 24-bit BMP and reports everything else through err, like an image
// Windows cannot decode (the trainer leaves such an image out: engine/src/train_job.h:304).
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>

#include "image_io.h"

namespace {
std::string native_path(std::string p) {
    for (char& c : p)
        if (c == '\\') c = '/';
    return p;
}
uint32_t le32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | ((uint32_t)p[3] << 24); }

bool read_ppm(const std::string& bytes, int& w, int& h, std::vector<uint8_t>& rgb, std::string& err) {
    // "P6" <ws> width <ws> height <ws> maxval <one ws byte> raster; '#' starts a comment up to the end of the line
    size_t at = 2;
    long field[3];
    for (int i = 0; i < 3; i++) {
        for (;;) {
            while (at < bytes.size() && isspace((unsigned char)bytes[at])) at++;
            if (at < bytes.size() && bytes[at] == '#') { while (at < bytes.size() && bytes[at] != '\n') at++; continue; }
            break;
        }
        long v = 0;
        size_t digits = 0;
        while (at < bytes.size() && isdigit((unsigned char)bytes[at])) { v = v * 10 + (bytes[at++] - '0'); digits++; }
        if (!digits) { err = "bad PPM header"; return false; }
        field[i] = v;
    }
    at++;   // the single whitespace byte before the raster
    if (field[0] <= 0 || field[1] <= 0 || field[2] != 255) { err = "unsupported PPM (8-bit P6 only)"; return false; }
    const size_t n = (size_t)field[0] * field[1] * 3;
    if (bytes.size() < at + n) { err = "truncated PPM"; return false; }
    w = (int)field[0]; h = (int)field[1];
    rgb.assign(bytes.begin() + at, bytes.begin() + at + n);
    return true;
}

bool read_bmp(const std::string& bytes, int& w, int& h, std::vector<uint8_t>& rgb, std::string& err) {
    const uint8_t* b = (const uint8_t*)bytes.data();
    if (bytes.size() < 54) { err = "truncated BMP"; return false; }
    const uint32_t off = le32(b + 10);
    const int32_t bw = (int32_t)le32(b + 18), bh = (int32_t)le32(b + 22);
    const int bpp = b[28] | (b[29] << 8);
    if (bpp != 24 || le32(b + 30) != 0 || bw <= 0 || bh == 0) { err = "unsupported BMP (uncompressed 24-bit only)"; return false; }
    const int rows = bh < 0 ? -bh : bh;
    const size_t pitch = ((size_t)bw * 3 + 3) & ~(size_t)3;
    if (bytes.size() < off + pitch * rows) { err = "truncated BMP"; return false; }
    w = bw; h = rows;
    rgb.resize((size_t)w * h * 3);
    for (int y = 0; y < rows; y++) {
        const uint8_t* src = b + off + pitch * (bh < 0 ? y : rows - 1 - y);   // bottom-up unless the height is negative
        uint8_t* dst = rgb.data() + (size_t)y * w * 3;
        for (int x = 0; x < w; x++) { dst[3 * x] = src[3 * x + 2]; dst[3 * x + 1] = src[3 * x + 1]; dst[3 * x + 2] = src[3 * x]; }
    }
    return true;
}
}  // namespace

bool load_image_rgb(const std::string& path, int& w, int& h, std::vector<uint8_t>& rgb, std::string& err) {
    std::ifstream f(native_path(path), std::ios::binary);
    if (!f) { err = "cannot open " + path; return false; }
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string bytes = ss.str();
    if (bytes.size() >= 2 && bytes[0] == 'P' && bytes[1] == '6') return read_ppm(bytes, w, h, rgb, err);
    if (bytes.size() >= 2 && bytes[0] == 'B' && bytes[1] == 'M') return read_bmp(bytes, w, h, rgb, err);
    err = "no decoder for this image format in the POSIX build (PPM P6 and 24-bit BMP only)";
    return false;
}
