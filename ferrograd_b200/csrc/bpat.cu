// `.bpat` tensor files: the reference's checkpoint format (crates/fused_gpu/src/io/headers.rs:16-117;
// writers and readers crates/fused_gpu/src/io/versions/v0_v2.rs:60-139, v1.rs:40-150, :160-290).
//
//   v0   "bpat"        u8 count | per tensor: u64 ndim, u64 shape[ndim], f64 data
//   v1   "BPATv1\0\0"  as v0, plus per tensor u32 CRC-32 of (ndim, shape, data) and a trailing u32 CRC-32
//                      of every byte before it
//   v1m  "BPATv1m\0"   as v1 with u32 ndim, u32 shape, f32 data
//   v2   "BPAT\0f32"   u8 count | per tensor: u32 ndim, u32 shape[ndim], f32 data (no checksums)
//        "BPAT\0f16", "BPATbf16": the same with f16 / bf16 data (headers.rs:60-98; io/mod.rs:170-183)
// All little endian.  Reading accepts all six (f64 data is narrowed to f32; 16-bit files load into 16-bit
// tensors, as the reference's init_tensor_f16 / init_tensor_bf16 do); writing produces v2-f32, v2-f16, v2-bf16
// or v1m.  The reference's v1m WRITER emits 8-byte shape entries
// after a 4-byte ndim (v1.rs:83-96) although its reader and the documented layout use 4-byte entries
// (v1.rs:281-288, headers.rs:41-58); this implementation follows the documented layout.
#include <stdio.h>

#include <algorithm>
#include <new>
#include <string>
#include <vector>

#include "fg_internal.cuh"

namespace {

uint32_t crc_table[256];
bool crc_ready = false;
void crc_init() {
    if (crc_ready) return;
    for (uint32_t i = 0; i < 256; ++i) {
        uint32_t c = i;
        for (int k = 0; k < 8; ++k) c = (c & 1u) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
        crc_table[i] = c;
    }
    crc_ready = true;
}
// Running CRC-32 (IEEE, the polynomial crc32fast uses); start with 0.
uint32_t crc_update(uint32_t crc, const void* data, size_t n) {
    crc_init();
    const unsigned char* p = (const unsigned char*)data;
    crc = ~crc;
    for (size_t i = 0; i < n; ++i) crc = crc_table[(crc ^ p[i]) & 0xFFu] ^ (crc >> 8);
    return ~crc;
}

struct Entry {
    std::vector<uint32_t> shape;
    uint64_t numel;
    uint64_t offset;     // of the data in the file
};

const char* kMagic[6] = {"bpat", "BPATv1\0\0", "BPATv1m\0", "BPAT\0f32", "BPAT\0f16", "BPATbf16"};
const size_t kMagicLen[6] = {4, 8, 8, 8, 8, 8};
// bytes per stored element
inline size_t elem_bytes(int format) {
    return (format == FG_BPAT_V0 || format == FG_BPAT_V1) ? 8 : (format == FG_BPAT_V2_F16 || format == FG_BPAT_V2_BF16) ? 2 : 4;
}

}  // namespace

struct fg_bpat_file {
    std::string path;
    int format;
    std::vector<Entry> entries;
};

extern "C" {

int32_t fg_bpat_save(fg_ctx* ctx, const char* path, int32_t format, uint32_t count, fg_buf* const* tensors,
                     const uint32_t* ndims, const uint32_t* const* shapes) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, path && (count == 0 || (tensors && ndims && shapes)), "fg_bpat_save: NULL argument");
    FG_REQUIRE(ctx, format == FG_BPAT_V2_F32 || format == FG_BPAT_V1_MICRO || format == FG_BPAT_V2_F16 || format == FG_BPAT_V2_BF16,
               "fg_bpat_save: only v2-f32, v2-f16, v2-bf16 and v1m can be written");
    FG_REQUIRE(ctx, count <= 255, "fg_bpat_save: exceeds max tensors of 255");
    const size_t esz_out = elem_bytes(format);
    for (uint32_t t = 0; t < count; ++t) {
        uint64_t n = 1;
        for (uint32_t d = 0; d < ndims[t]; ++d) n *= shapes[t][d];
        // the tensors must already have the file's storage type (the reference writes the buffer's bytes as they are)
        FG_REQUIRE(ctx, tensors[t] && tensors[t]->bytes == n * esz_out, "fg_bpat_save: tensor prod(shape)/data.size mismatch");
    }
    FILE* f = fopen(path, "wb");
    if (!f) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_bpat_save: cannot open the file for writing");
    const bool crc = format == FG_BPAT_V1_MICRO;
    uint32_t file_crc = 0;
    bool ok = true;
    auto put = [&](const void* p, size_t n, uint32_t* tensor_crc) {
        ok = ok && fwrite(p, 1, n, f) == n;
        file_crc = crc_update(file_crc, p, n);
        if (tensor_crc) *tensor_crc = crc_update(*tensor_crc, p, n);
    };
    put(kMagic[format], kMagicLen[format], nullptr);
    const uint8_t cnt = (uint8_t)count;
    put(&cnt, 1, nullptr);
    std::vector<char> host;
    int32_t status = FG_OK;
    for (uint32_t t = 0; t < count && ok; ++t) {
        uint32_t tcrc = 0;
        put(&ndims[t], 4, &tcrc);
        put(shapes[t], 4 * (size_t)ndims[t], &tcrc);
        host.resize(tensors[t]->bytes);
        status = fg_download(ctx, tensors[t], host.data(), tensors[t]->bytes, 0);
        if (status != FG_OK) break;
        put(host.data(), host.size(), &tcrc);
        if (crc) put(&tcrc, 4, nullptr);
    }
    if (status == FG_OK && ok && crc) {
        const uint32_t fc = file_crc;
        ok = fwrite(&fc, 1, 4, f) == 4;
    }
    ok = (fclose(f) == 0) && ok;
    if (status != FG_OK) return status;
    return ok ? FG_OK : fg_fail(ctx, FG_ERR_FAILED_BUFFER_COPY, "fg_bpat_save: failed to write to file");
}

// Parses the header and the tensor index, and verifies every checksum the format carries.
int32_t fg_bpat_open(const char* path, fg_bpat_file** out) {
    if (!path || !out) return FG_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    FILE* f = fopen(path, "rb");
    if (!f) return FG_ERR_INVALID_ARGUMENT;   // ErrorKind::FileNotFound
    unsigned char magic[8] = {0};
    int format = -1;
    if (fread(magic, 1, 4, f) == 4 && memcmp(magic, "bpat", 4) == 0) format = FG_BPAT_V0;
    else if (fread(magic + 4, 1, 4, f) == 4) {
        for (int k = 1; k < 6; ++k) if (memcmp(magic, kMagic[k], 8) == 0) format = k;
    }
    if (format < 0) { fclose(f); return FG_ERR_INVALID_ARGUMENT; }
    fg_bpat_file* bf = new (std::nothrow) fg_bpat_file();
    if (!bf) { fclose(f); return FG_ERR_OUT_OF_MEMORY; }
    bf->path = path;
    bf->format = format;
    const bool wide = format == FG_BPAT_V0 || format == FG_BPAT_V1;     // u64 ndim/shape, f64 data
    const bool crc = format == FG_BPAT_V1 || format == FG_BPAT_V1_MICRO;
    const size_t isz = wide ? 8 : 4, esz = elem_bytes(format);
    uint32_t file_crc = crc_update(0, magic, kMagicLen[format]);
    bool ok = true;
    auto get = [&](void* p, size_t n, uint32_t* tcrc) {
        ok = ok && fread(p, 1, n, f) == n;
        if (ok) { file_crc = crc_update(file_crc, p, n); if (tcrc) *tcrc = crc_update(*tcrc, p, n); }
    };
    uint8_t count = 0;
    get(&count, 1, nullptr);
    std::vector<char> chunk(1 << 20);
    for (uint32_t t = 0; t < count && ok; ++t) {
        uint32_t tcrc = 0;
        uint64_t ndim = 0;
        get(&ndim, isz, &tcrc);
        if (!ok || ndim > 8) { ok = false; break; }
        Entry e;
        e.numel = 1;
        for (uint64_t d = 0; d < ndim && ok; ++d) {
            uint64_t v = 0;
            get(&v, isz, &tcrc);
            e.shape.push_back((uint32_t)v);
            e.numel *= v;
        }
        e.offset = (uint64_t)ftell(f);
        uint64_t left = e.numel * esz;
        if (crc) {
            while (left && ok) { size_t n = (size_t)std::min<uint64_t>(left, chunk.size()); get(chunk.data(), n, &tcrc); left -= n; }
            uint32_t stored = 0;
            get(&stored, 4, nullptr);
            if (ok && stored != tcrc) ok = false;     // per-tensor checksum
        } else {
            ok = ok && fseek(f, (long)left, SEEK_CUR) == 0;
        }
        bf->entries.push_back(e);
    }
    if (ok && crc) {
        const uint32_t expect = file_crc;
        uint32_t stored = 0;
        ok = fread(&stored, 1, 4, f) == 4 && stored == expect;   // whole-file checksum
    }
    if (ok && !crc) {   // the data of the last tensor must actually be there
        const long pos = ftell(f);
        fseek(f, 0, SEEK_END);
        ok = ftell(f) >= pos;
    }
    fclose(f);
    if (!ok) { delete bf; return FG_ERR_FAILED_BUFFER_COPY; }   // SerializationError: truncated or corrupt
    *out = bf;
    return FG_OK;
}

int32_t fg_bpat_close(fg_bpat_file* f) { delete f; return FG_OK; }
int32_t fg_bpat_format(const fg_bpat_file* f) { return f ? f->format : -1; }
// Storage type of the tensors fg_bpat_load_tensor returns for this file.
int32_t fg_bpat_dtype(const fg_bpat_file* f) {
    if (!f) return -1;
    return f->format == FG_BPAT_V2_F16 ? FG_DTYPE_F16 : f->format == FG_BPAT_V2_BF16 ? FG_DTYPE_BF16 : FG_DTYPE_F32;
}
uint32_t fg_bpat_count(const fg_bpat_file* f) { return f ? (uint32_t)f->entries.size() : 0; }

int32_t fg_bpat_shape(const fg_bpat_file* f, uint32_t index, uint32_t* ndim, uint32_t dims_out[8]) {
    if (!f || !ndim || !dims_out || index >= f->entries.size()) return FG_ERR_INVALID_ARGUMENT;
    *ndim = (uint32_t)f->entries[index].shape.size();
    for (uint32_t d = 0; d < *ndim; ++d) dims_out[d] = f->entries[index].shape[d];
    return FG_OK;
}

// Allocates a device buffer and fills it with tensor `index`: f32, or the file's 16-bit type (init_tensor_*,
// dispatch/mod.rs:577-655).
int32_t fg_bpat_load_tensor(fg_ctx* ctx, const fg_bpat_file* f, uint32_t index, fg_buf** out) {
    if (!ctx) return FG_ERR_NOT_INITIALIZED;
    FG_REQUIRE(ctx, f && out && index < f->entries.size(), "fg_bpat_load_tensor: bad argument");
    const Entry& e = f->entries[index];
    const bool wide = f->format == FG_BPAT_V0 || f->format == FG_BPAT_V1;
    FILE* fp = fopen(f->path.c_str(), "rb");
    if (!fp) return fg_fail(ctx, FG_ERR_INVALID_ARGUMENT, "fg_bpat_load_tensor: file not found");
    if (elem_bytes(f->format) == 2) {
        // a 16-bit file loads into a 16-bit tensor, bytes unchanged (init_tensor_f16 / init_tensor_bf16)
        std::vector<uint16_t> half(e.numel);
        const bool ok16 = fseek(fp, (long)e.offset, SEEK_SET) == 0 && fread(half.data(), 2, e.numel, fp) == e.numel;
        fclose(fp);
        if (!ok16) return fg_fail(ctx, FG_ERR_FAILED_BUFFER_COPY, "fg_bpat_load_tensor: failed to read the tensor data");
        return fg_alloc_init(ctx, half.data(), e.numel * 2, out);
    }
    std::vector<float> host(e.numel);
    bool ok = fseek(fp, (long)e.offset, SEEK_SET) == 0;
    if (ok && !wide) ok = fread(host.data(), 4, e.numel, fp) == e.numel;
    if (ok && wide) {
        std::vector<double> wide_host(e.numel);
        ok = fread(wide_host.data(), 8, e.numel, fp) == e.numel;
        for (uint64_t i = 0; ok && i < e.numel; ++i) host[i] = (float)wide_host[i];
    }
    fclose(fp);
    if (!ok) return fg_fail(ctx, FG_ERR_FAILED_BUFFER_COPY, "fg_bpat_load_tensor: failed to read the tensor data");
    return fg_alloc_init(ctx, host.data(), e.numel * 4, out);
}

}  // extern "C"
