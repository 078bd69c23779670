/*
 * slab_loader.h — routed-expert weights straight from the engine's weight
 * container into HBM (host code only).
 *
 * The engine's eager load resolves each expert's two tensors by name and
 * concatenates them into two 1.5 GiB host arrays per layer (c/model.h:505-537)
 * before anything can use them.  On disk, though, an expert already is one
 * contiguous record — the "slab" {gate_up [2I,H] | down [H,I]}, 6 291 456 bytes
 * on the real model — located by the manifest apus.index.json, whose
 * expert_slabs array holds {layer, expert, shard, offset, nbytes} and whose
 * format_version must be 2 (c/cache.h:13-23,1000-1060).  This loader reads the
 * slabs of ONE layer's resident expert range through two pinned staging
 * buffers and copies each into the layer's exp_gu / exp_d tensors, so a rank
 * of an expert-parallel server touches only its own experts and no
 * whole-layer host copy is ever made.
 *
 * The manifest also carries a large tensor_map; the scanner below walks the
 * JSON text once, skipping every value it does not need.
 */
#pragma once
#include <cuda_runtime.h>
#include <fcntl.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace apus {

struct SlabRec {
    long layer = -1, expert = -1;
    std::string shard;
    uint64_t offset = 0, nbytes = 0;
};

/* minimal JSON walker: enough to find two top-level members */
struct JsonScan {
    const char *p, *end;
    bool ok = true;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
    }
    bool eat(char c) {
        ws();
        if (p < end && *p == c) {
            p++;
            return true;
        }
        return false;
    }
    std::string str() {
        std::string s;
        ws();
        if (p >= end || *p != '"') {
            ok = false;
            return s;
        }
        p++;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                p++;
                s.push_back(*p == 'n' ? '\n' : (*p == 't' ? '\t' : *p));   /* \uXXXX kept raw */
            } else {
                s.push_back(*p);
            }
            p++;
        }
        if (p >= end) ok = false;
        p++;
        return s;
    }
    double num() {
        ws();
        char *e = nullptr;
        double v = strtod(p, &e);
        if (e == p) ok = false;
        p = e;
        return v;
    }
    void skip() {               /* any value */
        ws();
        if (p >= end) {
            ok = false;
            return;
        }
        if (*p == '"') {
            str();
        } else if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            p++;
            if (eat(close)) return;
            do {
                if (open == '{') {
                    str();
                    if (!eat(':')) ok = false;
                }
                skip();
            } while (ok && eat(','));
            if (!eat(close)) ok = false;
        } else {
            while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n')
                p++;
        }
    }
};

/* expert_slabs of a manifest text; false (with a message) on malformed JSON, a
 * missing array, or format_version != 2 */
inline bool parse_manifest(const std::string &text, std::vector<SlabRec> *out, char *err,
                           size_t errcap) {
    JsonScan j{text.data(), text.data() + text.size()};
    long version = -1;
    bool have_slabs = false;
    if (!j.eat('{')) {
        snprintf(err, errcap, "manifest: not a JSON object");
        return false;
    }
    if (!j.eat('}')) {
        do {
            const std::string key = j.str();
            if (!j.eat(':')) j.ok = false;
            if (key == "format_version") {
                version = (long)j.num();
            } else if (key == "expert_slabs") {
                have_slabs = true;
                if (!j.eat('[')) j.ok = false;
                if (!j.eat(']')) {
                    do {
                        SlabRec r;
                        if (!j.eat('{')) j.ok = false;
                        if (!j.eat('}')) {
                            do {
                                const std::string k = j.str();
                                if (!j.eat(':')) j.ok = false;
                                if (k == "layer") r.layer = (long)j.num();
                                else if (k == "expert") r.expert = (long)j.num();
                                else if (k == "shard") r.shard = j.str();
                                else if (k == "offset") r.offset = (uint64_t)j.num();
                                else if (k == "nbytes") r.nbytes = (uint64_t)j.num();
                                else j.skip();
                            } while (j.ok && j.eat(','));
                            if (!j.eat('}')) j.ok = false;
                        }
                        out->push_back(r);
                    } while (j.ok && j.eat(','));
                    if (!j.eat(']')) j.ok = false;
                }
            } else {
                j.skip();
            }
        } while (j.ok && j.eat(','));
    }
    if (!j.ok) {
        snprintf(err, errcap, "manifest: malformed JSON near byte %ld",
                 (long)(j.p - text.data()));
        return false;
    }
    if (version != 2) {
        snprintf(err, errcap,
                 "manifest: format_version %ld != 2 (this loader reads the two-member "
                 "fused slab gate_up|down)", version);
        return false;
    }
    if (!have_slabs) {
        snprintf(err, errcap, "manifest: no expert_slabs array");
        return false;
    }
    return true;
}

/* Read the slabs of `layer_index` for experts [e_begin, e_end) from `dir` into
 * d_gu [(e_end-e_begin), 2I, H] and d_d [(e_end-e_begin), H, I].  Synchronous.
 * Returns the bytes uploaded, or -1 with a message. */
inline long long load_layer_slabs(const char *dir, int layer_index, size_t e_begin,
                                  size_t e_end, size_t H, size_t I, uint16_t *d_gu,
                                  uint16_t *d_d, char *err, size_t errcap) {
    const std::string path = std::string(dir) + "/apus.index.json";
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) {
        snprintf(err, errcap, "cannot open %s", path.c_str());
        return -1;
    }
    std::string text;
    char buf[1 << 16];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, n);
    fclose(f);
    std::vector<SlabRec> recs;
    if (!parse_manifest(text, &recs, err, errcap)) return -1;
    const size_t gu_bytes = 2 * I * H * 2, d_bytes = H * I * 2, slab = gu_bytes + d_bytes;
    const size_t ne = e_end - e_begin;
    std::vector<const SlabRec *> want(ne, nullptr);
    for (const SlabRec &r : recs)
        if (r.layer == layer_index && r.expert >= (long)e_begin && r.expert < (long)e_end)
            want[(size_t)r.expert - e_begin] = &r;
    for (size_t i = 0; i < ne; i++) {
        if (!want[i]) {
            snprintf(err, errcap, "manifest: no slab record for layer %d expert %zu",
                     layer_index, e_begin + i);
            return -1;
        }
        if (want[i]->nbytes != slab) {
            snprintf(err, errcap, "slab of layer %d expert %zu is %llu bytes, expected %zu",
                     layer_index, e_begin + i, (unsigned long long)want[i]->nbytes, slab);
            return -1;
        }
    }
    /* two pinned staging buffers: the copy of one slab overlaps the read of the next */
    unsigned char *stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaStream_t st = nullptr;
    long long total = -1;
    int fd = -1;
    std::string open_shard;
    bool ok = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;
    for (int b = 0; ok && b < 2; b++)
        ok = cudaMallocHost((void **)&stage[b], slab) == cudaSuccess &&
             cudaEventCreateWithFlags(&done[b], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) snprintf(err, errcap, "slab loader: pinned staging allocation failed");
    for (size_t i = 0; ok && i < ne; i++) {
        const SlabRec &r = *want[i];
        const int b = (int)(i & 1);
        if (i >= 2 && cudaEventSynchronize(done[b]) != cudaSuccess) {
            snprintf(err, errcap, "slab loader: copy failed");
            ok = false;
            break;
        }
        if (r.shard != open_shard) {
            if (fd >= 0) close(fd);
            const std::string sp = std::string(dir) + "/" + r.shard;
            fd = open(sp.c_str(), O_RDONLY);
            if (fd < 0) {
                snprintf(err, errcap, "cannot open shard %s", sp.c_str());
                ok = false;
                break;
            }
            open_shard = r.shard;
        }
        size_t got = 0;
        while (got < slab) {
            const ssize_t k = pread(fd, stage[b] + got, slab - got, (off_t)(r.offset + got));
            if (k <= 0) break;
            got += (size_t)k;
        }
        if (got != slab) {
            snprintf(err, errcap, "short read of layer %d expert %zu in %s", layer_index,
                     e_begin + i, r.shard.c_str());
            ok = false;
            break;
        }
        ok = cudaMemcpyAsync(d_gu + i * 2 * I * H, stage[b], gu_bytes, cudaMemcpyHostToDevice,
                             st) == cudaSuccess &&
             cudaMemcpyAsync(d_d + i * H * I, stage[b] + gu_bytes, d_bytes,
                             cudaMemcpyHostToDevice, st) == cudaSuccess &&
             cudaEventRecord(done[b], st) == cudaSuccess;
        if (!ok) snprintf(err, errcap, "slab loader: upload failed");
    }
    if (ok && cudaStreamSynchronize(st) != cudaSuccess) {
        snprintf(err, errcap, "slab loader: upload failed");
        ok = false;
    }
    if (ok) total = (long long)(ne * slab);
    if (fd >= 0) close(fd);
    for (int b = 0; b < 2; b++) {
        if (done[b]) cudaEventDestroy(done[b]);
        if (stage[b]) cudaFreeHost(stage[b]);
    }
    if (st) cudaStreamDestroy(st);
    return total;
}

}  // namespace apus
