// GGUF file -> device: the raw blocks of one tensor go from the file to their place in a GGUF-block map
// without passing through Python objects.  Replaces the reference's load loop (adam/loaders/gguf.py:196-253
// load_tensor_raw / iter_tensor_chunks feeding adam/models/engine.py:929-1116, which decodes every chunk to
// float32 on the host and re-quantizes it with per-group Python loops).
//
// The tensor is read in chunks of whole blocks (32 MB, the reference's max_chunk_mb) into two pinned host
// buffers; each chunk is one cudaMemcpyAsync, so the read of chunk i+1 overlaps the copy (and, for the types kept
// in planes, the repack kernel) of chunk i.  Q4_K keeps the file layout and is copied straight to its place.
#include "blocks8.cuh"

#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <unistd.h>

namespace ab {

constexpr size_t FILE_CHUNK = 32u << 20;
struct FileStage { void* pinned[2]; void* dev[2]; cudaEvent_t done[2]; bool ok; };
static FileStage s_fs = {};

static int file_stage_prepare() {
    if (s_fs.ok) return ADAMAH_OK;
    for (int i = 0; i < 2; ++i) {
        if (cudaMallocHost(&s_fs.pinned[i], FILE_CHUNK) != cudaSuccess || cudaMalloc(&s_fs.dev[i], FILE_CHUNK) != cudaSuccess ||
            cudaEventCreateWithFlags(&s_fs.done[i], cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return fail(ADAMAH_ERR_MEMORY, "file upload: cannot allocate the staging buffers");
        }
    }
    s_fs.ok = true;
    return ADAMAH_OK;
}
void file_stage_release() {
    for (int i = 0; i < 2; ++i) {
        if (s_fs.pinned[i]) cudaFreeHost(s_fs.pinned[i]);
        if (s_fs.dev[i]) cudaFree(s_fs.dev[i]);
        if (s_fs.done[i]) cudaEventDestroy(s_fs.done[i]);
    }
    s_fs = FileStage{};
}

}  // namespace ab

using namespace ab;

extern "C" int adam_b200_upload_gguf_file(uint32_t map_wt, uint32_t ggml_type, uint64_t elem_off, const char* path, uint64_t file_offset, uint64_t n_bytes) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    Map* m = get_map(map_wt);
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!path || n_bytes == 0) return fail(ADAMAH_ERR_INVALID, "upload_gguf_file: empty input");
    const BlockKind* k = block_kind(ggml_type);
    int rc = check_block_range(m, map_wt, k, ggml_type, elem_off, n_bytes);
    if (rc) return rc;
    if ((rc = file_stage_prepare())) return rc;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(ADAMAH_ERR_INVALID, "upload_gguf_file: cannot open %s: %s", path, strerror(errno));
    posix_fadvise(fd, (off_t)file_offset, (off_t)n_bytes, POSIX_FADV_SEQUENTIAL);
    const size_t chunk = FILE_CHUNK / k->bytes * k->bytes;          // whole blocks
    uint64_t done = 0;
    for (int i = 0; done < n_bytes && rc == ADAMAH_OK; ++i) {
        const int s = i & 1;
        const size_t take = n_bytes - done < chunk ? (size_t)(n_bytes - done) : chunk;
        if (i >= 2 && cudaEventSynchronize(s_fs.done[s]) != cudaSuccess) { rc = fail(ADAMAH_ERR_BACKEND, "upload_gguf_file: staging wait failed"); break; }
        size_t got = 0;
        while (got < take) {
            const ssize_t r = pread(fd, (char*)s_fs.pinned[s] + got, take - got, (off_t)(file_offset + done + got));
            if (r < 0 && errno == EINTR) continue;
            if (r <= 0) { rc = fail(ADAMAH_ERR_INVALID, "upload_gguf_file: %s ends %llu bytes short of the tensor", path, (unsigned long long)(n_bytes - done - got)); break; }
            got += (size_t)r;
        }
        if (rc) break;
        const uint64_t e_off = elem_off + done / k->bytes * k->elems;
        if (ggml_type == 12) {
            if (cudaMemcpyAsync((uint8_t*)m->buf + e_off / 256 * 144, s_fs.pinned[s], take, cudaMemcpyHostToDevice, g.stream) != cudaSuccess) rc = fail(ADAMAH_ERR_BACKEND, "upload_gguf_file: copy failed");
        } else {
            if (cudaMemcpyAsync(s_fs.dev[s], s_fs.pinned[s], take, cudaMemcpyHostToDevice, g.stream) != cudaSuccess) rc = fail(ADAMAH_ERR_BACKEND, "upload_gguf_file: copy failed");
            else rc = place_blocks_from_device(m, *k, e_off, s_fs.dev[s], take);
        }
        cudaEventRecord(s_fs.done[s], g.stream);
        done += take;
    }
    close(fd);
    if (cudaStreamSynchronize(g.stream) != cudaSuccess && rc == ADAMAH_OK) rc = fail(ADAMAH_ERR_BACKEND, "upload_gguf_file: %s", cudaGetErrorString(cudaGetLastError()));
    return rc ? rc : check_launch("adam_b200_upload_gguf_file");
}
