#include "llava_device_memory.h"

#include <algorithm>
#include <iostream>
#include <vector>

#include "llava_buffer.h"
#include "llava_context.h"

using namespace std;

llava_device_memory::llava_device_memory(llava_context* _context) : context(_context) {}

llava_device_memory::~llava_device_memory() {
    if (!buffers.empty()) cerr << "[?] device memory destroyed while " << buffers.size() << " buffers still use it" << endl;
    if (base) lv_arena_free(context->lv(), base);
}

bool llava_device_memory::freeze() {
    if (is_frozen()) return false;
    void* p = nullptr;
    if (lv_arena_create(context->lv(), max<size_t>(cursor, 256), &p) != LV_OK) {
        cerr << "[!] device allocation of " << cursor << " bytes failed: " << lv_last_error_string() << endl;
        return false;
    }
    base = static_cast<u8*>(p);
    return true;
}

void llava_device_memory::register_llava_buffer(llava_buffer* buffer) {
    if (!buffers.insert(buffer).second) cerr << "[?] A buffer was registered twice to a device memory" << endl;
}

void llava_device_memory::forget_llava_buffer(llava_buffer* buffer) { buffers.erase(buffer); }

size_t llava_device_memory::register_buffer(size_t alignment, size_t buffer_size) {
    if (alignment == 0) alignment = 1;
    cursor = (cursor + alignment - 1) / alignment * alignment;
    const size_t at = cursor;
    cursor += buffer_size;
    return at;
}

bool llava_device_memory::write(size_t offset, const void* src, size_t size) const {
    return is_frozen() && offset + size <= cursor && lv_upload(context->lv(), base + offset, src, size) == LV_OK;
}

bool llava_device_memory::read(size_t offset, void* dst, size_t size) const {
    return is_frozen() && offset + size <= cursor && lv_download(context->lv(), dst, base + offset, size) == LV_OK;
}

bool llava_device_memory::zero(size_t offset, size_t size) const {
    return is_frozen() && offset + size <= cursor && lv_memset(context->lv(), base + offset, 0, size) == LV_OK;
}

void llava_device_memory::dump_buffers(int out_fd, const string& name) {
    // llava_device_memory.cpp:80-97 of the reference walks a set ordered by pointer; sorting
    // by name makes the frame file reproducible
    vector<llava_buffer*> ordered(buffers.begin(), buffers.end());
    sort(ordered.begin(), ordered.end(), [](llava_buffer* a, llava_buffer* b) { return a->get_pretty_name() < b->get_pretty_name(); });
    for (llava_buffer* b : ordered) {
        const string& pretty = b->get_pretty_name();
        if (pretty.empty() || pretty == "k_cache" || pretty == "v_cache") continue;
        b->dump_raw(out_fd, name + "." + pretty);
    }
}
