// TEST INFRASTRUCTURE - NOT PRODUCT CODE.
//
// C-ABI doors onto the REFERENCE's own strixw writer and reader (strixite formats/strixw.cpp), which build.py compiles
// unchanged from the mounted reference tree into oracle/_ref/libstrix_formats_ref.so. No format logic lives here: the
// functions only build the reference's structs from flat arguments. Used to pin strixite_b200/strixw.py both ways:
// a file written by the reference's StrixwWriter is what tests/golden/demo.strixw holds, and a file written by this
// repository's writer must open and hash-verify under the reference's StrixwFile.

#include "formats/strixw.hpp"

#include <cstdint>
#include <cstring>
#include <exception>
#include <map>
#include <string>
#include <vector>

namespace {
thread_local std::string g_msg;

// Deterministic filler: byte i of component (tensor ti, role r) = a fixed function of (seed, ti, r, i), restated in
// tests/golden/make_golden.py so that the test can regenerate the expected bytes.
void fill(std::vector<uint8_t> &b, uint64_t seed, uint64_t ti, uint64_t role) {
    uint64_t s = seed * 0x9e3779b97f4a7c15ull + ti * 0x100000001b3ull + role * 0xd6e8feb86659fd93ull + 1;
    for (size_t i = 0; i < b.size(); ++i) {
        s ^= s << 13, s ^= s >> 7, s ^= s << 17;  // xorshift64
        b[i] = (uint8_t)(s >> 32);
    }
}
}  // namespace

extern "C" {

const char *ref_strixw_last_error() { return g_msg.c_str(); }

uint64_t ref_hash64(const void *p, uint64_t n) { return strix::strix_hash64(p, (size_t)n); }

// Writes the demonstration file: one tensor of every row-major encoding the MoE path loads, an expert stack with parts,
// metadata. Shapes are small; component bytes come from fill().
int ref_strixw_write_demo(const char *path, uint64_t seed) {
    try {
        using namespace strix;
        std::vector<StrixwTensor> ts;
        auto add = [&](const char *name, StrixwEncoding e, std::vector<int64_t> shape, int64_t G, int64_t experts) {
            StrixwTensor t;
            t.name = name, t.encoding = e, t.shape = std::move(shape), t.group_size = G, t.experts = experts;
            ts.push_back(std::move(t));
        };
        add("layers.0.moe.router", StrixwEncoding::BF16, {5, 128}, 0, 0);
        add("layers.0.moe.experts.gate_up", StrixwEncoding::Q4RowMajor, {3 * 64, 128}, 32, 3);
        ts.back().parts = {{"model.layers.0.mlp.experts.gate_up_proj", 0, 128}, {"model.layers.0.mlp.shared_expert.gate_up", 128, 64}};
        add("layers.0.moe.experts.down", StrixwEncoding::Q5RowMajor, {3 * 128, 128}, 128, 3);
        add("layers.0.moe.shared.down", StrixwEncoding::Q8RowMajor, {128, 64}, 64, 0);
        add("layers.0.moe.shared.gate_up", StrixwEncoding::Q6RowMajor, {64, 128}, 64, 0);
        add("norm.weight", StrixwEncoding::F32, {128}, 0, 0);
        add("positions", StrixwEncoding::I64, {2, 3}, 0, 0);
        std::map<std::string, std::string> meta = {{"model", "demo"}, {"converter", "reference StrixwWriter"}, {"empty", ""}};
        StrixwWriter w(path, meta, ts);
        for (size_t ti = 0; ti < w.tensors().size(); ++ti)
            for (const StrixwComponent &c : w.tensors()[ti].components) {
                std::vector<uint8_t> b(c.bytes);
                fill(b, seed, ti, (uint64_t)c.role);
                w.write(ti, c.role, b.data(), b.size());
            }
        w.finish();
        return 0;
    } catch (const std::exception &e) {
        g_msg = e.what();
        return 1;
    }
}

// Opens a file with the reference's reader, verifies every hash, and reports the number of tensors and the file size.
int ref_strixw_check(const char *path, int64_t *n_tensors, uint64_t *file_bytes) {
    try {
        strix::StrixwFile f(path);
        f.verify_hashes(2);
        *n_tensors = (int64_t)f.tensors().size();
        *file_bytes = f.file_bytes();
        return 0;
    } catch (const std::exception &e) {
        g_msg = e.what();
        return 1;
    }
}

}  // extern "C"
