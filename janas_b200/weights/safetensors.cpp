#include "safetensors.h"

#include <cerrno>
#include <cstring>
#include <fcntl.h>
#include <fstream>
#include <set>
#include <sstream>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "../core/json.h"

namespace jb {

[[noreturn]] static void bad(const std::string &m) { throw Error(JB_LLM_EOPEN, m); }

int stored_size(const std::string &dt) {
    if (dt == "F32" || dt == "I32") return 4;
    if (dt == "F16" || dt == "BF16") return 2;
    if (dt == "I64") return 8;
    return 0;
}

SafetensorsFile::SafetensorsFile(const std::string &p) : path(p) {
    struct stat st;
    if (stat(p.c_str(), &st) != 0) bad(p + ": " + strerror(errno));
    size_ = (size_t)st.st_size;
    if (size_ < 8) bad(p + ": too short for a safetensors header");
    fd_ = ::open(p.c_str(), O_RDONLY);
    if (fd_ < 0) bad(p + ": " + strerror(errno));
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (map_ == MAP_FAILED) {
        map_ = nullptr;
        int e = errno;
        ::close(fd_);
        fd_ = -1;
        bad(p + ": cannot be mapped: " + strerror(e));
    }
    const uint8_t *base = (const uint8_t *)map_;
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | base[i];
    if (hlen < 2 || hlen > size_ - 8)
        bad(fmt("%s: header length %llu does not fit the file (%zu bytes)", p.c_str(),
                (unsigned long long)hlen, size_));
    Json header;
    try {
        header = Json::parse(std::string((const char *)base + 8, (size_t)hlen));
    } catch (const JsonError &e) {
        bad(p + ": the header is not JSON (" + e.what() + ")");
    }
    if (!header.is_object()) bad(p + ": the header is not a JSON object");
    size_t data_start = 8 + (size_t)hlen;
    for (auto &m : header.members()) {
        const std::string &name = m.first;
        if (name == "__metadata__") continue;
        const Json &ent = m.second;
        const Json &dt = ent.get("dtype"), &sh = ent.get("shape"), &off = ent.get("data_offsets");
        bool ok = ent.is_object() && dt.is_string() && sh.is_array() && off.is_array() &&
                  off.size() == 2 && off[0].is_number() && off[1].is_number();
        if (ok)
            for (auto &s : sh.items()) ok = ok && s.is_number() && s.whole();
        if (!ok) bad(p + ": malformed entry for " + name);
        int esz = stored_size(dt.as_string());
        if (!esz)
            bad(p + ": tensor " + name + " has dtype " + dt.as_string() +
                ", which is not read (F32, F16, BF16, I32, I64)");
        TensorInfo t;
        t.name = name;
        t.dtype = dt.as_string();
        bool neg = false;
        unsigned __int128 count = 1;
        for (auto &s : sh.items()) {
            long long v = s.as_int();
            neg |= v < 0;
            t.shape.push_back(v);
            count *= (unsigned __int128)(v < 0 ? 0 : v);
        }
        long long b = off[0].as_int(), e = off[1].as_int();
        if (neg || b < 0 || e < b || (unsigned __int128)(e - b) != count * (unsigned)esz ||
            (unsigned long long)e > size_ - data_start) {
            std::string shp = "[";
            for (size_t i = 0; i < t.shape.size(); i++)
                shp += (i ? ", " : "") + std::to_string(t.shape[i]);
            shp += "]";
            bad(fmt("%s: tensor %s: its byte range [%lld, %lld) does not match shape %s %s or lies "
                    "outside the file", p.c_str(), name.c_str(), b, e, shp.c_str(), t.dtype.c_str()));
        }
        t.begin = data_start + (size_t)b;
        t.end = data_start + (size_t)e;
        t.path = p;
        t.data = base + t.begin;
        tensors.push_back(std::move(t));
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
}

static bool is_file(const std::string &p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

void Checkpoint::open_file(const std::string &path) {
    files_.emplace_back(new SafetensorsFile(path));
    for (auto &t : files_.back()->tensors) {
        auto it = tensors.find(t.name);
        if (it != tensors.end()) bad(path + ": tensor " + t.name + " is also in " + it->second.path);
        tensors[t.name] = t;
        names.push_back(t.name);
    }
}

Checkpoint::Checkpoint(const std::string &dir) : model_dir(dir) {
    std::string index = dir + "/model.safetensors.index.json";
    std::string single = dir + "/model.safetensors";
    if (is_file(index)) {
        std::ifstream f(index, std::ios::binary);
        std::stringstream ss;
        ss << f.rdbuf();
        Json j;
        try {
            j = Json::parse(ss.str());
        } catch (const JsonError &) {
            bad(index + ": no weight_map");
        }
        const Json &wm = j.get("weight_map");
        if (!wm.is_object()) bad(index + ": no weight_map");
        std::set<std::string> fnames;
        for (auto &m : wm.members()) {
            if (!m.second.is_string()) bad(index + ": no weight_map");
            fnames.insert(m.second.as_string());
        }
        for (auto &fn : fnames) {
            if (fn.find('/') != std::string::npos || fn.find("..") != std::string::npos)
                bad(index + ": a shard outside the folder: " + fn);
            open_file(dir + "/" + fn);
        }
        for (auto &m : wm.members()) {
            auto it = tensors.find(m.first);
            if (it == tensors.end() || it->second.path != dir + "/" + m.second.as_string())
                bad(index + ": " + m.first + " is not in " + m.second.as_string());
        }
    } else if (is_file(single)) {
        open_file(single);
    } else {
        bad(dir + ": no model.safetensors (nor model.safetensors.index.json)");
    }
}

}  // namespace jb
