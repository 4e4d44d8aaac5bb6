// Reads a .safetensors file (8-byte little-endian header length, JSON header, raw tensor data) and
// hands every entry to lumi_model_load_tensor — the same file the reference maps with
// VarBuilder::from_mmaped_safetensors (inference/src/main.rs:83-85).
#include "internal.h"
#include "json_min.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>

using namespace lumi;

extern "C" int32_t lumi_model_load_safetensors(lumi_model* m, const char* path) {
    if (!m || !path) return fail(LUMI_E_INVALID, "null argument to lumi_model_load_safetensors");
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(LUMI_E_IO, "cannot open '%s'", path);
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 8) { close(fd); return fail(LUMI_E_IO, "'%s' is too short to be a safetensors file", path); }
    const size_t size = (size_t)sb.st_size;
    void* map = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return fail(LUMI_E_IO, "mmap of '%s' failed", path);
    const uint8_t* base = (const uint8_t*)map;
    uint64_t hlen = 0;
    memcpy(&hlen, base, 8);
    int32_t status = LUMI_OK;
    if (hlen == 0 || hlen > size - 8) {
        status = fail(LUMI_E_IO, "'%s': header length %llu exceeds the file", path, (unsigned long long)hlen);
    } else {
        JsonValue root;
        std::string err;
        JsonParser p((const char*)base + 8, (size_t)hlen);
        if (!p.parse(root, err) || root.kind != JsonValue::Object) {
            status = fail(LUMI_E_IO, "'%s': malformed header: %s", path, err.c_str());
        } else {
            const uint8_t* data = base + 8 + hlen;
            const size_t data_size = size - 8 - (size_t)hlen;
            for (auto& kv : root.obj) {
                if (kv.first == "__metadata__") continue;
                const JsonValue& e = kv.second;
                const JsonValue* dt = e.find("dtype");
                const JsonValue* sh = e.find("shape");
                const JsonValue* off = e.find("data_offsets");
                if (!dt || !sh || !off || dt->kind != JsonValue::String || sh->kind != JsonValue::Array ||
                    off->kind != JsonValue::Array || off->arr.size() != 2) {
                    status = fail(LUMI_E_IO, "'%s': entry '%s' lacks dtype / shape / data_offsets", path, kv.first.c_str());
                    break;
                }
                int dtype;
                if (dt->str == "F32") dtype = LUMI_DTYPE_F32;
                else if (dt->str == "BF16") dtype = LUMI_DTYPE_BF16;
                else {
                    if (kv.first.rfind("item.", 0) != 0) continue;
                    status = fail(LUMI_E_TENSOR, "tensor '%s': dtype %s not supported (F32, BF16)", kv.first.c_str(), dt->str.c_str());
                    break;
                }
                int64_t shape[8];
                int rank = 0;
                for (auto& d : sh->arr) { if (rank < 8) shape[rank++] = (int64_t)d.num; }
                const uint64_t b0 = (uint64_t)off->arr[0].num, b1 = (uint64_t)off->arr[1].num;
                if (b1 < b0 || b1 > data_size) {
                    status = fail(LUMI_E_IO, "'%s': entry '%s' points outside the file", path, kv.first.c_str());
                    break;
                }
                status = lumi_model_load_tensor(m, kv.first.c_str(), dtype, shape, rank, data + b0, b1 - b0);
                if (status != LUMI_OK) break;
            }
        }
    }
    munmap(map, size);
    return status;
}
