// CPU-only: runs the reference's own model loaders (Dit::load, TextEncoder::load, Vae::load) on a models directory with the
// weight upload replaced by a stub that only records shapes, and prints what the loaders saw. Linked against the engine's
// object files with this definition of upload_weight taking precedence; no CUDA call is made.
#include <cstdio>

#include "models.h"

Weight upload_weight(const StTensor& t, Place, bool temporal_last, bool f16) {
    Weight w;
    if (t.shape.empty()) { w.rows = 1; w.cols = 1; }
    else {
        w.rows = t.shape[0];
        int64_t rest = 1;
        for (size_t i = 1; i < t.shape.size(); i++) if (!(temporal_last && i == 2)) rest *= t.shape[i];
        w.cols = rest;
    }
    if (temporal_last && t.shape.size() != 5) printf("bad temporal kernel (%zu dims)\n", t.shape.size());
    if ((size_t)t.numel() * 2 != t.bytes) printf("bad byte count\n");
    w.p = (uint16_t*)0x1000;      // non-null: "loaded"; never dereferenced
    w.f16 = f16;
    return w;
}

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    const std::string dir = argv[1];
    try {
        Vae v;
        v.load(dir + "\\qwen_image_vae.safetensors", Place::Device);
        printf("vae top %ld stages %zu %zu fp16 %d\n", (long)v.conv1.rows, v.ups.size(), v.downs.size(), (int)v.use_fp16());
        for (auto& u : v.ups) { printf("up %d:", u.cout); for (auto& r : u.res) printf(" %d>%d%s", r.cin, r.cout, r.sc ? "s" : ""); printf(" rs %ldx%ld\n", (long)u.rs.rows, (long)u.rs.cols); }
        for (auto& d : v.downs) { printf("down %d:", d.cout); for (auto& r : d.res) printf(" %d>%d%s", r.cin, r.cout, r.sc ? "s" : ""); printf(" ds %ldx%ld\n", (long)d.ds.rows, (long)d.ds.cols); }
        printf("vae head %ldx%ld ehead %ldx%ld q %ldx%ld\n", (long)v.head_c.rows, (long)v.head_c.cols, (long)v.e_head_c.rows, (long)v.e_head_c.cols,
               (long)v.q_conv.rows, (long)v.q_conv.cols);
        Dit d;
        d.load(dir + "\\anima-base-v1.0.safetensors", Place::Device);
        printf("dit named %zu prefix %s blocks %zu adapter %zu\n", d.named.size(), d.prefix.c_str(), d.blocks.size(), d.ad_blocks.size());
        for (auto& nw : d.named)
            if (nw.first.rfind("blocks.0.", 0) == 0 || nw.first.find("blocks.") == std::string::npos || nw.first.rfind("llm_adapter.blocks.0.", 0) == 0)
                printf("w %s %ldx%ld\n", nw.first.c_str(), (long)nw.second->rows, (long)nw.second->cols);
        TextEncoder t;
        t.load(dir + "\\qwen_3_06b_base.safetensors", Place::Device);
        printf("te layers %zu ff %ld vocab %ld q %ldx%ld k %ldx%ld o %ldx%ld\n", t.layers.size(), (long)t.layers[0].gate.rows, (long)t.embed->shape[0],
               (long)t.layers[0].q.rows, (long)t.layers[0].q.cols, (long)t.layers[0].k.rows, (long)t.layers[0].k.cols, (long)t.layers[0].o.rows,
               (long)t.layers[0].o.cols);
    } catch (const std::exception& e) {
        printf("FAILED %s\n", e.what());
        return 1;
    }
    return 0;
}
