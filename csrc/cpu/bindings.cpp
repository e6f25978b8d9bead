// Python bindings of the CPU oracle (module sketchml_b200._oracle).
#include <pybind11/numpy.h>
#include <algorithm>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "oracle.h"

namespace py = pybind11;
using namespace skml;

typedef py::array_t<int32_t, py::array::c_style | py::array::forcecast> I32Array;
typedef py::array_t<double, py::array::c_style | py::array::forcecast> F64Array;
typedef py::array_t<float, py::array::c_style | py::array::forcecast> F32Array;
typedef py::array_t<uint64_t, py::array::c_style | py::array::forcecast> U64Array;

template <class T>
static py::array_t<T> to_array(const std::vector<T>& v) {
    py::array_t<T> a(v.size());
    if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
    return a;
}

static py::bytes to_bytes(const std::vector<uint8_t>& b) {
    return py::bytes(reinterpret_cast<const char*>(b.data()), b.size());
}

static bool is_f32(const py::array& a) { return a.dtype().is(py::dtype::of<float>()); }

static SketchOptions options_from(const py::dict& d) {
    SketchOptions o;
    auto geti = [&](const char* k, auto& dst) {
        if (d.contains(k)) dst = d[k].cast<std::decay_t<decltype(dst)>>();
    };
    geti("bin_num", o.bin_num);
    geti("group_num", o.group_num);
    geti("row_num", o.row_num);
    geti("col_ratio", o.col_ratio);
    geti("key_encoder", o.key_encoder);
    geti("cell_bits", o.cell_bits);
    geti("sketch_k", o.sketch_k);
    geti("threads", o.threads);
    geti("seed", o.seed);
    geti("step", o.step);
    geti("rank", o.rank);
    geti("world", o.world);
    geti("offset_mode", o.offset_mode);
    geti("tie_mode", o.tie_mode);
    geti("java_compat_max", o.java_compat_max);
    geti("restart", o.restart);
    if (d.contains("loss_partials")) {
        auto lp = d["loss_partials"].cast<std::vector<double>>();
        for (size_t i = 0; i < lp.size() && i < 4; ++i) o.loss_partials[i] = lp[i];
    }
    return o;
}

template <class T>
static py::dict quantizer_dict(const Quantizer<T>& q) {
    py::dict r;
    r["bin_num"] = q.bin_num;
    r["zero_idx"] = q.zero_idx;
    r["min"] = (double)q.min;
    r["max"] = (double)q.max;
    r["splits"] = to_array(q.splits);
    r["bins"] = to_array(q.bins);
    r["values"] = to_array(q.values());
    return r;
}

static py::dict encoded_dict(const EncodedKeys& e) {
    py::dict r;
    r["size"] = e.size;
    r["num_intervals"] = e.num_intervals;
    r["flag_kind"] = e.flag_kind;
    r["flag_words"] = to_array(e.flags.words);
    r["delta_words"] = to_array(e.deltas.words);
    r["flag_bits"] = e.flag_bits;
    r["delta_bits"] = e.delta_bits;
    return r;
}

static EncodedKeys encoded_from(const py::dict& d) {
    EncodedKeys e;
    e.size = d["size"].cast<uint32_t>();
    e.num_intervals = d["num_intervals"].cast<uint32_t>();
    e.flag_kind = d["flag_kind"].cast<uint32_t>();
    e.flags.words = d["flag_words"].cast<std::vector<uint64_t>>();
    e.deltas.words = d["delta_words"].cast<std::vector<uint64_t>>();
    return e;
}

template <class T>
struct PySketch {
    QuantileSketch<T> s;
    PySketch(int k, uint64_t seed, int offset_mode, bool jmax) : s(k, seed, offset_mode, jmax) {}
};

template <class T>
static py::dict parse_payload(const std::string& buf) {
    SketchGradient<T> g = skml_parse<T>(reinterpret_cast<const uint8_t*>(buf.data()), buf.size());
    py::dict r;
    const SkmlHeader& h = g.h;
    r["kind"] = h.kind;
    r["dtype"] = h.dtype;
    r["step"] = h.step;
    r["rank"] = h.rank;
    r["world"] = h.world;
    r["dim"] = h.dim;
    r["nnz"] = h.nnz;
    r["bin_num"] = h.bin_num;
    r["zero_idx"] = h.zero_idx;
    r["group_num"] = h.group_num;
    r["row_num"] = h.row_num;
    r["col_ratio"] = h.col_ratio;
    r["key_encoder"] = h.key_encoder;
    r["cell_bits"] = h.cell_bits;
    r["seed"] = h.seed;
    r["min_value"] = h.min_value;
    r["max_value"] = h.max_value;
    r["restart_interval"] = h.restart_interval;
    r["total_bytes"] = h.total_bytes;
    r["loss_partials"] = std::vector<double>(h.loss_partials, h.loss_partials + 4);
    py::dict offs;
    offs["bucket_values"] = h.off_bucket_values;
    offs["group_table"] = h.off_group_table;
    offs["tables"] = h.off_tables;
    offs["key_flags"] = h.off_key_flags;
    offs["key_deltas"] = h.off_key_deltas;
    offs["restart"] = h.off_restart;
    offs["dense_codes"] = h.off_dense_codes;
    r["offsets"] = offs;
    r["bucket_values"] = to_array(g.bucket_values);
    if (h.kind == SKML_KIND_DENSE) {
        r["dense_codes"] = to_array(g.dense_codes);
    } else if (h.kind == SKML_KIND_SPARSE) {
        py::list groups;
        std::vector<SkmlGroupEntry> ent(h.group_num);
        std::memcpy(ent.data(), buf.data() + h.off_group_table, h.group_num * sizeof(SkmlGroupEntry));
        for (uint32_t i = 0; i < h.group_num; ++i) {
            py::dict gd;
            const MinMaxSketch& m = g.sketch.sketches[i];
            gd["n"] = ent[i].n;
            gd["col_num"] = ent[i].col_num;
            gd["hash_ids"] = std::vector<int>(ent[i].hash_ids, ent[i].hash_ids + 8);
            gd["table_off"] = ent[i].table_off;
            gd["flag_off"] = ent[i].flag_off;
            gd["delta_off"] = ent[i].delta_off;
            gd["restart_off"] = ent[i].restart_off;
            gd["n_flag_words"] = ent[i].n_flag_words;
            gd["n_delta_words"] = ent[i].n_delta_words;
            gd["table"] = to_array(m.table);
            gd["keys"] = encoded_dict(g.sketch.keys[i]);
            if (ent[i].n && ent[i].restart_off) {
                size_t cnt = (ent[i].n + h.restart_interval - 1) / h.restart_interval;
                std::vector<uint64_t> raw(cnt * 2);
                std::memcpy(raw.data(), buf.data() + ent[i].restart_off, cnt * 16);
                gd["restart_raw"] = to_array(raw);
            }
            groups.append(gd);
        }
        r["groups"] = groups;
        r["edges"] = g.sketch.edges;
    }
    return r;
}

// ---------------------------------------------------------------------------
// Native text parser: one pass over the bytes of a libsvm / csv / dummy file slice.
// Formats as in the reference's ml/data/Parser.scala:23-76 (libsvm "label idx:val ...",
// csv "label,v,v,...", dummy "label,idx,idx,..." with implicit 1.0 values); labels that are not
// within 1e-8 of 1 become -1 when neg_y is set. Columns of a row are sorted and duplicate
// columns merged (values add up).
// ---------------------------------------------------------------------------
static py::tuple parse_text(const std::string& text, const std::string& fmt, long long max_dim, bool neg_y) {
    const int kind = fmt == "libsvm" ? 0 : (fmt == "csv" ? 1 : (fmt == "dummy" ? 2 : -1));
    if (kind < 0) throw Error("Unknown file format: " + fmt);
    std::vector<int64_t> rowptr{0};
    std::vector<int32_t> cols;
    std::vector<double> vals, labels;
    std::vector<std::pair<int32_t, double>> row;
    const char* p = text.data();
    const char* end = p + text.size();
    bool dup = false;
    while (p < end) {
        const char* eol = static_cast<const char*>(memchr(p, '\n', end - p));
        if (!eol) eol = end;
        const char* q = p;
        while (q < eol && (*q == ' ' || *q == '\t' || *q == '\r')) ++q;
        if (q < eol) {
            char* next = nullptr;
            double y = strtod(q, &next);
            if (next == q) throw Error("cannot parse label in line: " + std::string(p, std::min<size_t>(eol - p, 60)));
            if (neg_y && std::fabs(y - 1.0) > 1e-8) y = -1.0;
            q = next;
            row.clear();
            int dense_i = 0;
            while (q < eol) {
                while (q < eol && (*q == ' ' || *q == ',' || *q == '\t' || *q == '\r')) ++q;
                if (q >= eol) break;
                if (kind == 0) {
                    long idx = strtol(q, &next, 10);
                    if (next == q || next >= eol || *next != ':') throw Error("expected idx:val in line: " + std::string(p, std::min<size_t>(eol - p, 60)));
                    q = next + 1;
                    double v = strtod(q, &next);
                    if (next == q) throw Error("expected a value after ':'");
                    q = next;
                    row.push_back({(int32_t)idx, v});
                } else if (kind == 1) {
                    double v = strtod(q, &next);
                    if (next == q) throw Error("cannot parse csv value");
                    q = next;
                    row.push_back({dense_i++, v});
                } else {
                    long idx = strtol(q, &next, 10);
                    if (next == q) throw Error("cannot parse feature index");
                    q = next;
                    row.push_back({(int32_t)idx, 1.0});
                }
            }
            std::stable_sort(row.begin(), row.end(), [](const auto& a, const auto& b) { return a.first < b.first; });
            int32_t last = -1;
            for (auto& kv : row) {
                if (kv.first < 0 || kv.first >= max_dim)
                    throw Error("feature index out of range [0, " + std::to_string(max_dim) + ")");
                if (kv.first == last) {
                    vals.back() += kv.second;
                    dup = true;
                } else {
                    cols.push_back(kv.first);
                    vals.push_back(kv.second);
                    last = kv.first;
                }
            }
            labels.push_back(y);
            rowptr.push_back((int64_t)cols.size());
        }
        p = eol + 1;
    }
    return py::make_tuple(to_array(rowptr), to_array(cols), to_array(vals), to_array(labels), kind == 2 && !dup);
}

PYBIND11_MODULE(_oracle, m) {
    m.def("parse_text", &parse_text, py::arg("text"), py::arg("format"), py::arg("max_dim"), py::arg("neg_y") = true);
    m.doc() = "CPU oracle of the SketchML compression algorithms";
    py::register_exception<Error>(m, "SketchMLError");

    m.def("hash", [](int id, I32Array keys, int32_t size) {
        if (id < 0 || id > 7) throw Error("hash id out of range [0, 8)");
        if (size <= 0) throw Error("hash range must be positive");
        std::vector<int32_t> out(keys.size());
        for (ssize_t i = 0; i < keys.size(); ++i) out[i] = skml_hash(id, keys.data()[i], size);
        return to_array(out);
    });
    m.def("hash_fast", [](int id, I32Array keys, int32_t size) {
        if (id < 0 || id > 7 || size <= 0) throw Error("hash id or range out of bounds");
        std::vector<int32_t> out(keys.size());
        uint64_t magic = skml_fastmod_magic((uint32_t)size);
        for (ssize_t i = 0; i < keys.size(); ++i) {
            SkmlKeyDigits kd;
            skml_key_digits(keys.data()[i], kd);
            out[i] = skml_hash_fast(id, keys.data()[i], kd, size, magic);
        }
        return to_array(out);
    });
    m.def("hash_rows", [](std::vector<int> ids, I32Array keys, int32_t size) {
        // the kernels' multi-row hash (one shared digit pass): returns [len(keys)][len(ids)]
        if (ids.empty() || ids.size() > 8 || size <= 0) throw Error("hash ids or range out of bounds");
        uint8_t id8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (size_t r = 0; r < ids.size(); ++r) {
            if (ids[r] < 0 || ids[r] > 7) throw Error("hash id out of range [0, 8)");
            id8[r] = (uint8_t)ids[r];
        }
        const int rows = (int)ids.size();
        std::vector<int32_t> out((size_t)keys.size() * rows);
        uint64_t magic = skml_fastmod_magic((uint32_t)size);
        for (ssize_t i = 0; i < keys.size(); ++i) {
            int32_t pos[8];
            if (rows <= 4) skml_hash_rows<4>(id8, rows, keys.data()[i], size, magic, pos);
            else skml_hash_rows<8>(id8, rows, keys.data()[i], size, magic, pos);
            for (int r = 0; r < rows; ++r) out[(size_t)i * rows + r] = pos[r];
        }
        return to_array(out);
    });
    m.def("pack_bits", [](I32Array v, int bits) {
        // Little-endian bit stream: value i occupies stream bits [i * bits, (i + 1) * bits), stream bit b is
        // bit (b & 31) of 32-bit word b >> 5. Two zero words of padding follow so that a reader may always
        // fetch the word after the one a value starts in.
        if (bits < 1 || bits > 32) throw Error("pack_bits: bits out of range [1, 32]");
        const size_t n = (size_t)v.size();
        const size_t words = (n * (size_t)bits + 31) / 32 + 2;
        std::vector<uint32_t> out(words, 0u);
        const uint64_t mask = bits == 32 ? 0xFFFFFFFFull : ((1ull << bits) - 1ull);
        for (size_t i = 0; i < n; ++i) {
            const uint64_t x = (uint64_t)(uint32_t)v.data()[i];
            if (x & ~mask) throw Error("pack_bits: value does not fit in " + std::to_string(bits) + " bits");
            const size_t bit = i * (size_t)bits, w = bit >> 5;
            const unsigned sh = (unsigned)(bit & 31);
            const uint64_t wide = x << sh;
            out[w] |= (uint32_t)wide;
            out[w + 1] |= (uint32_t)(wide >> 32);
        }
        return to_array(out);
    }, py::arg("values"), py::arg("bits"));
    m.def("unpack_bits", [](py::array_t<uint32_t, py::array::c_style | py::array::forcecast> w, size_t n, int bits) {
        if (bits < 1 || bits > 32) throw Error("unpack_bits: bits out of range [1, 32]");
        if ((n * (size_t)bits + 31) / 32 + 1 > (size_t)w.size()) throw Error("unpack_bits: stream too short");
        std::vector<int32_t> out(n);
        const uint64_t mask = bits == 32 ? 0xFFFFFFFFull : ((1ull << bits) - 1ull);
        for (size_t i = 0; i < n; ++i) {
            const size_t bit = i * (size_t)bits, k = bit >> 5;
            const uint64_t wide = (uint64_t)w.data()[k] | ((uint64_t)w.data()[k + 1] << 32);
            out[i] = (int32_t)((wide >> (bit & 31)) & mask);
        }
        return to_array(out);
    }, py::arg("words"), py::arg("n"), py::arg("bits"));
    m.def("pack_varbytes", [](I32Array v) {
        // Byte-aligned variable-width code for non-negative integers: value i takes 1..4 little-endian
        // bytes (the fewest that hold it); its width - 1 sits in bits [2 (i & 15), 2 (i & 15) + 2) of
        // 32-bit flag word i >> 4; `block_offsets[b]` is the byte offset of value 1024 b, so that blocks
        // of 1024 values decode independently. The byte stream ends with 24 bytes of padding (a reader fetches five aligned words per 4 values).
        const size_t n = (size_t)v.size();
        std::vector<uint32_t> flags((n + 15) / 16 + 1, 0u);
        std::vector<uint32_t> offs((n + 1023) / 1024 + 1, 0u);
        std::vector<uint8_t> bytes;
        bytes.reserve(n * 2 + 16);
        for (size_t i = 0; i < n; ++i) {
            if ((i & 1023) == 0) offs[i >> 10] = (uint32_t)bytes.size();
            const int32_t sv = v.data()[i];
            if (sv < 0) throw Error("pack_varbytes: negative value");
            const uint32_t x = (uint32_t)sv;
            const int w = x < (1u << 8) ? 1 : (x < (1u << 16) ? 2 : (x < (1u << 24) ? 3 : 4));
            flags[i >> 4] |= (uint32_t)(w - 1) << (2 * (i & 15));
            for (int j = 0; j < w; ++j) bytes.push_back((uint8_t)(x >> (8 * j)));
            if (bytes.size() > 0xFFFFFF00ull) throw Error("pack_varbytes: stream too long");
        }
        offs[(n + 1023) / 1024] = (uint32_t)bytes.size();
        bytes.resize(bytes.size() + 24, 0);
        py::dict r;
        r["flags"] = to_array(flags);
        r["block_offsets"] = to_array(offs);
        r["bytes"] = to_array(bytes);
        return r;
    }, py::arg("values"));
    m.def("unpack_varbytes", [](py::array_t<uint32_t, py::array::c_style | py::array::forcecast> flags,
                                py::array_t<uint8_t, py::array::c_style | py::array::forcecast> bytes, size_t n) {
        std::vector<int32_t> out(n);
        size_t pos = 0;
        for (size_t i = 0; i < n; ++i) {
            if ((i >> 4) >= (size_t)flags.size()) throw Error("unpack_varbytes: flags too short");
            const int w = (int)((flags.data()[i >> 4] >> (2 * (i & 15))) & 3u) + 1;
            if (pos + w > (size_t)bytes.size()) throw Error("unpack_varbytes: bytes too short");
            uint32_t x = 0;
            for (int j = 0; j < w; ++j) x |= (uint32_t)bytes.data()[pos + j] << (8 * j);
            out[i] = (int32_t)x;
            pos += w;
        }
        return to_array(out);
    }, py::arg("flags"), py::arg("bytes"), py::arg("n"));
    m.def("pack_varnibbles", [](I32Array v) {
        // Nibble-aligned variable-width code for non-negative integers: value i takes 1..8 nibbles (the
        // fewest that hold it), lowest nibble first, nibble p of the stream in bits [4 (p & 7), +4) of 32-bit
        // word p >> 3; its width - 1 sits in 3 flag bits at bit 3 i of the flag stream (same word order);
        // `block_offsets[b]` is the nibble offset of value 1024 b. Both streams end with padding words.
        const size_t n = (size_t)v.size();
        std::vector<uint32_t> flags((3 * n + 31) / 32 + 2, 0u);
        std::vector<uint32_t> offs((n + 1023) / 1024 + 1, 0u);
        std::vector<uint32_t> words;
        words.reserve(n / 2 + 16);
        uint64_t nib = 0;
        for (size_t i = 0; i < n; ++i) {
            if ((i & 1023) == 0) offs[i >> 10] = (uint32_t)nib;
            const int32_t sv = v.data()[i];
            if (sv < 0) throw Error("pack_varnibbles: negative value");
            const uint32_t x = (uint32_t)sv;
            int w = 1;
            while (w < 8 && (x >> (4 * w)) != 0) ++w;
            const size_t fb = 3 * i;
            const uint64_t fw = (uint64_t)(w - 1) << (fb & 31);
            flags[fb >> 5] |= (uint32_t)fw;
            flags[(fb >> 5) + 1] |= (uint32_t)(fw >> 32);
            const size_t bit = (size_t)nib * 4, wi = bit >> 5;
            if (words.size() < wi + 2) words.resize(wi + 2, 0u);
            const uint64_t wide = (uint64_t)x << (bit & 31);
            words[wi] |= (uint32_t)wide;
            words[wi + 1] |= (uint32_t)(wide >> 32);
            nib += (uint64_t)w;
            if (nib > 0xFFFFFF00ull) throw Error("pack_varnibbles: stream too long");
        }
        offs[(n + 1023) / 1024] = (uint32_t)nib;
        words.resize((size_t)((nib * 4 + 31) / 32) + 6, 0u);
        py::dict r;
        r["flags"] = to_array(flags);
        r["block_offsets"] = to_array(offs);
        r["words"] = to_array(words);
        return r;
    }, py::arg("values"));
    m.def("unpack_varnibbles", [](py::array_t<uint32_t, py::array::c_style | py::array::forcecast> flags,
                                  py::array_t<uint32_t, py::array::c_style | py::array::forcecast> words, size_t n) {
        std::vector<int32_t> out(n);
        uint64_t nib = 0;
        for (size_t i = 0; i < n; ++i) {
            const size_t fb = 3 * i;
            if ((fb >> 5) + 1 >= (size_t)flags.size()) throw Error("unpack_varnibbles: flags too short");
            const uint64_t fwide = (uint64_t)flags.data()[fb >> 5] | ((uint64_t)flags.data()[(fb >> 5) + 1] << 32);
            const int w = (int)((fwide >> (fb & 31)) & 7u) + 1;
            const size_t bit = (size_t)nib * 4, wi = bit >> 5;
            if (wi + 1 >= (size_t)words.size()) throw Error("unpack_varnibbles: words too short");
            const uint64_t wide = (uint64_t)words.data()[wi] | ((uint64_t)words.data()[wi + 1] << 32);
            const uint64_t x = wide >> (bit & 31);
            out[i] = (int32_t)(w == 8 ? (uint32_t)x : (uint32_t)(x & ((1ull << (4 * w)) - 1ull)));
            nib += (uint64_t)w;
        }
        return to_array(out);
    }, py::arg("flags"), py::arg("words"), py::arg("n"));
    m.def("row_sort_delta", [](py::array_t<int64_t, py::array::c_style | py::array::forcecast> rowptr, I32Array cols) {
        // Every row's indices sorted ascending and replaced by their gaps (the first one stays): the order
        // inside a row carries no information, and gaps between sorted indices are shorter than the indices.
        const ssize_t rows = rowptr.size() - 1;
        std::vector<int32_t> out(cols.data(), cols.data() + cols.size());
        for (ssize_t r = 0; r < rows; ++r) {
            const int64_t lo = rowptr.data()[r] - rowptr.data()[0], hi = rowptr.data()[r + 1] - rowptr.data()[0];
            if (lo < 0 || hi < lo || hi > (int64_t)out.size()) throw Error("row_sort_delta: bad row pointers");
            std::sort(out.begin() + lo, out.begin() + hi);
            int32_t prev = 0;
            for (int64_t e = lo; e < hi; ++e) {
                const int32_t v = out[e];
                out[e] = v - prev;
                prev = v;
            }
        }
        return to_array(out);
    }, py::arg("rowptr"), py::arg("cols"));
    m.def("pick_hashes", [](uint64_t seed, uint64_t step, uint32_t rank, uint32_t group, int rows) {
        if (rows > 8 || rows < 1) throw Error("Currently only 8 hash functions are available");
        uint8_t ids[8];
        skml_pick_hashes(seed, step, rank, group, rows, ids);
        return std::vector<int>(ids, ids + rows);
    });
    m.def("group_edges", [](int zero, int bins, int groups) {
        std::vector<int> e(groups);
        skml_group_edges(zero, bins, groups, e.data());
        return e;
    });
    m.def("rand64", [](uint64_t seed, uint64_t a, uint64_t b, uint64_t c) { return skml_rand(seed, a, b, c); });

    py::class_<PySketch<double>>(m, "QuantileSketch")
        .def(py::init<int, uint64_t, int, bool>(), py::arg("k") = 128, py::arg("seed") = 0,
             py::arg("offset_mode") = 2, py::arg("java_compat_max") = false)
        .def("update", [](PySketch<double>& s, F64Array v) {
            for (ssize_t i = 0; i < v.size(); ++i) s.s.update(v.data()[i]);
        })
        .def("merge", [](PySketch<double>& s, const PySketch<double>& o) { s.s.merge(o.s); })
        .def("quantiles", [](PySketch<double>& s, int q) { return to_array(s.s.quantiles(q)); })
        .def("summary", [](PySketch<double>& s) {
            std::vector<double> a;
            std::vector<uint64_t> c;
            s.s.summary(a, c);
            return py::make_tuple(to_array(a), to_array(c));
        })
        .def("reset", [](PySketch<double>& s) { s.s.reset(); })
        .def_property_readonly("n", [](PySketch<double>& s) { return s.s.n(); })
        .def_property_readonly("min", [](PySketch<double>& s) { return s.s.min_value(); })
        .def_property_readonly("max", [](PySketch<double>& s) { return s.s.max_value(); })
        .def_property_readonly("k", [](PySketch<double>& s) { return s.s.k(); })
        .def_property_readonly("retained", [](PySketch<double>& s) { return s.s.retained(); });

    m.def("quantile_quantize",
          [](py::array v, int bins, int k, uint64_t seed, int offset_mode, bool jmax, int threads) -> py::dict {
              if (is_f32(v)) {
                  F32Array a(v);
                  return quantizer_dict(quantile_quantize_parallel<float>(a.data(), a.size(), bins, k, seed, offset_mode, jmax, threads));
              }
              F64Array a(v);
              return quantizer_dict(quantile_quantize_parallel<double>(a.data(), a.size(), bins, k, seed, offset_mode, jmax, threads));
          },
          py::arg("values"), py::arg("bin_num") = 256, py::arg("k") = 128, py::arg("seed") = 0,
          py::arg("offset_mode") = 2, py::arg("java_compat_max") = false, py::arg("threads") = 1);
    m.def("uniform_quantize", [](F64Array v, int bins) {
        return quantizer_dict(uniform_quantize<double>(v.data(), v.size(), bins));
    });
    m.def("zipml_quantize", [](F64Array v, int bins) {
        return quantizer_dict(zipml_quantize<double>(v.data(), v.size(), bins));
    });
    m.def("quantizer_from_splits", [](py::array splits, double mn, double mx, py::array v) -> py::dict {
        if (is_f32(v)) {
            F32Array s(splits), a(v);
            std::vector<float> sv(s.data(), s.data() + s.size());
            return quantizer_dict(quantizer_from_splits<float>(sv, (float)mn, (float)mx, a.data(), a.size()));
        }
        F64Array s(splits), a(v);
        std::vector<double> sv(s.data(), s.data() + s.size());
        return quantizer_dict(quantizer_from_splits<double>(sv, mn, mx, a.data(), a.size()));
    });
    m.def("export_java_quantizer", [](F64Array splits, double mn, double mx, F64Array v) {
        std::vector<double> sv(splits.data(), splits.data() + splits.size());
        return to_bytes(export_java_quantizer(quantizer_from_splits<double>(sv, mn, mx, v.data(), v.size())));
    });

    m.def("delta_binary_encode", [](I32Array k) { return encoded_dict(delta_binary_encode(k.data(), k.size())); });
    m.def("delta_binary_decode", [](py::dict d) { return to_array(delta_binary_decode(encoded_from(d))); });
    m.def("delta_adaptive_encode", [](I32Array k) { return encoded_dict(delta_adaptive_encode(k.data(), k.size())); });
    m.def("delta_adaptive_decode", [](py::dict d) { return to_array(delta_adaptive_decode(encoded_from(d))); });
    m.def("set_bits", [](std::vector<uint64_t> words, uint64_t off, uint32_t value, int nbits) {
        BitStream b;
        b.words = words;
        b.put(off, value, nbits);
        return b.words;
    });
    m.def("get_bits", [](std::vector<uint64_t> words, uint64_t off, int nbits) {
        BitStream b;
        b.words = words;
        return b.take(off, nbits);
    });

    m.def("huffman_encode", [](I32Array v) {
        HuffmanCode h = huffman_encode(v.data(), v.size());
        py::dict r;
        py::list items;
        for (auto& it : h.items) items.append(py::make_tuple(it.value, it.bits, it.num_bits));
        r["items"] = items;
        r["words"] = to_array(h.bits.words);
        r["nbits"] = h.nbits;
        r["size"] = h.size;
        return r;
    });
    m.def("huffman_decode", [](py::dict d) {
        HuffmanCode h;
        h.size = d["size"].cast<uint32_t>();
        for (auto it : d["items"].cast<py::list>()) {
            auto t = it.cast<py::tuple>();
            h.items.push_back({t[0].cast<int32_t>(), t[1].cast<uint32_t>(), t[2].cast<int32_t>()});
        }
        h.bits.words = d["words"].cast<std::vector<uint64_t>>();
        return to_array(huffman_decode(h));
    });

    py::class_<MinMaxSketch>(m, "MinMaxSketch")
        .def(py::init([](int rows, int cols, int zero, std::vector<int> ids, int tie_mode) {
                 if (rows > 8) throw Error("Currently only 8 hash functions are available");
                 uint8_t h[8] = {0};
                 for (size_t i = 0; i < ids.size() && i < 8; ++i) h[i] = (uint8_t)ids[i];
                 return MinMaxSketch(rows, cols, zero, h, tie_mode);
             }),
             py::arg("rows"), py::arg("cols"), py::arg("zero"), py::arg("hash_ids"), py::arg("tie_mode") = 0)
        .def("insert", [](MinMaxSketch& s, I32Array k, I32Array b) {
            for (ssize_t i = 0; i < k.size(); ++i) s.insert(k.data()[i], b.data()[i]);
        })
        .def("query", [](MinMaxSketch& s, I32Array k) {
            std::vector<int32_t> r(k.size());
            for (ssize_t i = 0; i < k.size(); ++i) r[i] = s.query(k.data()[i]);
            return to_array(r);
        })
        .def_property_readonly("table", [](MinMaxSketch& s) { return to_array(s.table); });

    m.def("compress_sparse",
          [](I32Array keys, py::array vals, uint64_t dim, py::dict opts, py::object splits, double mn, double mx) {
              SketchOptions o = options_from(opts);
              if (keys.size() != vals.size()) throw Error("Lengths of key array and value array do not match");
              if (is_f32(vals)) {
                  F32Array a(vals);
                  if (splits.is_none()) return to_bytes(compress_sparse<float>(keys.data(), a.data(), a.size(), dim, o));
                  F32Array s(splits);
                  std::vector<float> sv(s.data(), s.data() + s.size());
                  return to_bytes(compress_sparse<float>(keys.data(), a.data(), a.size(), dim, o, &sv, (float)mn, (float)mx));
              }
              F64Array a(vals);
              if (splits.is_none()) return to_bytes(compress_sparse<double>(keys.data(), a.data(), a.size(), dim, o));
              F64Array s(splits);
              std::vector<double> sv(s.data(), s.data() + s.size());
              return to_bytes(compress_sparse<double>(keys.data(), a.data(), a.size(), dim, o, &sv, mn, mx));
          },
          py::arg("keys"), py::arg("values"), py::arg("dim"), py::arg("options"), py::arg("splits") = py::none(),
          py::arg("min") = 0.0, py::arg("max") = 0.0);
    m.def("compress_dense",
          [](py::array vals, py::dict opts, py::object splits, double mn, double mx) {
              SketchOptions o = options_from(opts);
              if (is_f32(vals)) {
                  F32Array a(vals);
                  if (splits.is_none()) return to_bytes(compress_dense<float>(a.data(), a.size(), o));
                  F32Array s(splits);
                  std::vector<float> sv(s.data(), s.data() + s.size());
                  return to_bytes(compress_dense<float>(a.data(), a.size(), o, &sv, (float)mn, (float)mx));
              }
              F64Array a(vals);
              if (splits.is_none()) return to_bytes(compress_dense<double>(a.data(), a.size(), o));
              F64Array s(splits);
              std::vector<double> sv(s.data(), s.data() + s.size());
              return to_bytes(compress_dense<double>(a.data(), a.size(), o, &sv, mn, mx));
          },
          py::arg("values"), py::arg("options"), py::arg("splits") = py::none(), py::arg("min") = 0.0,
          py::arg("max") = 0.0);
    m.def("payload_dtype", [](const std::string& b) {
        SkmlHeader h;
        skml_validate(reinterpret_cast<const uint8_t*>(b.data()), b.size(), h);
        return (int)h.dtype;
    });
    m.def("decompress", [](const std::string& b) {
        SkmlHeader h;
        const uint8_t* p = reinterpret_cast<const uint8_t*>(b.data());
        skml_validate(p, b.size(), h);
        std::vector<int32_t> keys;
        if (h.dtype == SKML_F32) {
            std::vector<float> v;
            decompress<float>(p, b.size(), keys, v);
            return py::make_tuple((int)h.kind, to_array(keys), py::array(to_array(v)));
        }
        std::vector<double> v;
        decompress<double>(p, b.size(), keys, v);
        return py::make_tuple((int)h.kind, to_array(keys), py::array(to_array(v)));
    });
    m.def("parse", [](const std::string& b) -> py::dict {
        SkmlHeader h;
        skml_validate(reinterpret_cast<const uint8_t*>(b.data()), b.size(), h);
        return h.dtype == SKML_F32 ? parse_payload<float>(b) : parse_payload<double>(b);
    });
    m.def("payload_times_by", [](const std::string& b, double x) {
        std::vector<uint8_t> c(b.begin(), b.end());
        payload_times_by(c.data(), c.size(), x);
        return to_bytes(c);
    });
    m.def("export_java_fields", [](const std::string& b) {
        SkmlHeader h;
        const uint8_t* p = reinterpret_cast<const uint8_t*>(b.data());
        skml_validate(p, b.size(), h);
        return to_bytes(h.dtype == SKML_F32 ? export_java_fields<float>(p, b.size())
                                            : export_java_fields<double>(p, b.size()));
    });

    m.def("fixed_point_encode", [](F64Array v, int bits, uint64_t seed) {
        FixedPointCode c = fixed_point_encode<double>(v.data(), v.size(), bits, seed);
        py::dict r;
        r["size"] = c.size;
        r["num_bits"] = c.num_bits;
        r["norm"] = c.norm;
        r["words"] = to_array(c.bits.words);
        return r;
    });
    m.def("fixed_point_decode", [](py::dict d) {
        FixedPointCode c;
        c.size = d["size"].cast<uint32_t>();
        c.num_bits = d["num_bits"].cast<int>();
        c.norm = d["norm"].cast<double>();
        c.bits.words = d["words"].cast<std::vector<uint64_t>>();
        return to_array(fixed_point_decode<double>(c));
    });

    m.def("quick_select", [](F64Array a, size_t k) {
        return quick_select(std::vector<double>(a.data(), a.data() + a.size()), k);
    });
    m.def("select_kth_largest", [](F64Array a, size_t k) {
        return select_kth_largest(std::vector<double>(a.data(), a.data() + a.size()), k);
    });
    m.def("kway_merge", [](std::vector<std::vector<int32_t>> ks, std::vector<std::vector<int32_t>> ys) {
        std::vector<int32_t> k, y;
        kway_merge(ks, ys, k, y);
        return py::make_tuple(to_array(k), to_array(y));
    });
    m.def("unique_sorted", [](F64Array a) {
        return to_array(unique_sorted(std::vector<double>(a.data(), a.data() + a.size())));
    });
    m.attr("HEADER_BYTES") = SKML_HEADER_BYTES;
    m.attr("RESTART_INTERVAL") = SKML_RESTART_INTERVAL;
}
