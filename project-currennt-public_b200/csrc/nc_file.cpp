// netCDF classic (CDF-1 / CDF-2) reader; see nc_file.hpp.
//
// Grammar (all integers big-endian, names and values padded to 4 bytes):
//   header   = "CDF" version(1|2) numrecs dim_list gatt_list var_list
//   dim_list = ABSENT | 0x0A nelems { name dim_length }            (dim_length 0 = record dimension)
//   att_list = ABSENT | 0x0C nelems { name nc_type nelems values }
//   var_list = ABSENT | 0x0B nelems { name ndims dimid* att_list nc_type vsize begin }
//   begin is 32 bits in CDF-1 and 64 bits in CDF-2; ABSENT = two zero words.
// Fixed-size variables are stored contiguously at `begin`; record variables are interleaved record
// by record, `recsize` (sum of their vsize) bytes apart.
#include "nc_file.hpp"

#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace b2 {
namespace {

inline uint32_t be32(const unsigned char *p) {
    return ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | (uint32_t)p[3];
}
inline uint64_t be64(const unsigned char *p) { return ((uint64_t)be32(p) << 32) | (uint64_t)be32(p + 4); }

int type_size(int t) {
    switch (t) {
        case NcFile::NC_BYTE: case NcFile::NC_CHAR: return 1;
        case NcFile::NC_SHORT: return 2;
        case NcFile::NC_INT: case NcFile::NC_FLOAT: return 4;
        case NcFile::NC_DOUBLE: return 8;
    }
    return 0;
}

// bounds-checked cursor over the header
struct Cursor {
    const unsigned char *p, *end;
    bool ok = true;
    uint32_t u32() {
        if (end - p < 4) { ok = false; return 0; }
        uint32_t v = be32(p);
        p += 4;
        return v;
    }
    uint64_t u64() {
        if (end - p < 8) { ok = false; return 0; }
        uint64_t v = be64(p);
        p += 8;
        return v;
    }
    std::string name() {
        uint32_t n = u32();
        size_t padded = ((size_t)n + 3) & ~(size_t)3;
        if (!ok || (size_t)(end - p) < padded) { ok = false; return std::string(); }
        std::string s((const char *)p, n);
        p += padded;
        return s;
    }
    void skip(size_t n) {
        if ((size_t)(end - p) < n) { ok = false; return; }
        p += n;
    }
    void att_list() {
        uint32_t tag = u32(), n = u32();
        if (!ok) return;
        if (tag == 0 && n == 0) return;
        if (tag != 0x0C) { ok = false; return; }
        for (uint32_t i = 0; i < n && ok; ++i) {
            name();
            uint32_t t = u32(), ne = u32();
            int ts = type_size((int)t);
            if (!ts) { ok = false; return; }
            skip((((size_t)ne * ts) + 3) & ~(size_t)3);
        }
    }
};

template <typename T>
inline T convert(const unsigned char *p, int type) {
    switch (type) {
        case NcFile::NC_FLOAT: {
            uint32_t u = be32(p);
            float f;
            memcpy(&f, &u, 4);
            return (T)f;
        }
        case NcFile::NC_DOUBLE: {
            uint64_t u = be64(p);
            double d;
            memcpy(&d, &u, 8);
            return (T)d;
        }
        case NcFile::NC_INT: return (T)(int32_t)be32(p);
        case NcFile::NC_SHORT: return (T)(int16_t)(((uint16_t)p[0] << 8) | p[1]);
        case NcFile::NC_BYTE: return (T)(int8_t)p[0];
    }
    return T();
}

}  // namespace

NcFile::~NcFile() { close(); }

void NcFile::close() {
    if (map_) munmap((void *)map_, size_);
    map_ = nullptr;
    size_ = 0;
    dims_.clear();
    vars_.clear();
}

std::string NcFile::open(const std::string &path) {
    close();
    path_ = path;
    int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) return "Could not open '" + path + "': " + strerror(errno);
    struct stat sb;
    if (fstat(fd, &sb) != 0 || sb.st_size < 32) {
        ::close(fd);
        return "Could not open '" + path + "': not a netCDF classic file";
    }
    size_ = (size_t)sb.st_size;
    void *m = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) {
        size_ = 0;
        return "Could not map '" + path + "': " + strerror(errno);
    }
    map_ = (const unsigned char *)m;
    if (memcmp(map_, "CDF", 3) != 0 || (map_[3] != 1 && map_[3] != 2)) {
        std::string why = (memcmp(map_, "\x89HDF", 4) == 0) ? "netCDF-4/HDF5 files are not supported (convert with nccopy -k classic)"
                                                             : "not a netCDF classic (CDF-1/CDF-2) file";
        close();
        return "Could not read '" + path + "': " + why;
    }
    version_ = map_[3];
    Cursor c{map_ + 4, map_ + size_};
    numrecs_ = c.u32();
    if (numrecs_ == 0xFFFFFFFFu) numrecs_ = 0;   // "streaming" marker: record count unknown
    // dimensions
    uint32_t tag = c.u32(), n = c.u32();
    if (c.ok && !(tag == 0 && n == 0)) {
        if (tag != 0x0A) c.ok = false;
        for (uint32_t i = 0; i < n && c.ok; ++i) {
            Dim d;
            d.name = c.name();
            d.len = c.u32();
            d.record = (d.len == 0);
            if (d.record) d.len = numrecs_;
            dims_.push_back(d);
        }
    }
    c.att_list();
    // variables
    tag = c.u32();
    n = c.u32();
    if (c.ok && !(tag == 0 && n == 0)) {
        if (tag != 0x0B) c.ok = false;
        for (uint32_t i = 0; i < n && c.ok; ++i) {
            Var v;
            v.name = c.name();
            uint32_t nd = c.u32();
            if (nd > 1024) c.ok = false;
            for (uint32_t k = 0; k < nd && c.ok; ++k) {
                uint32_t id = c.u32();
                if (id >= dims_.size()) c.ok = false;
                v.dimids.push_back((int)id);
            }
            c.att_list();
            v.type = (int)c.u32();
            v.vsize = c.u32();
            v.begin = (version_ == 2) ? c.u64() : c.u32();
            if (!c.ok || !type_size(v.type)) { c.ok = false; break; }
            v.record = !v.dimids.empty() && dims_[v.dimids[0]].record;
            v.rows = v.dimids.empty() ? 1 : dims_[v.dimids[0]].len;
            v.rowElems = 1;
            for (size_t k = 1; k < v.dimids.size(); ++k) v.rowElems *= dims_[v.dimids[k]].len;
            vars_.push_back(v);
        }
    }
    if (!c.ok) {
        close();
        return "Could not read '" + path + "': damaged netCDF header";
    }
    // record size: the sum of the record variables' vsize; a single record variable is stored
    // without padding between records
    int nrec = 0;
    recsize_ = 0;
    for (const Var &v : vars_)
        if (v.record) { ++nrec; recsize_ += v.vsize; }
    if (nrec == 1)
        for (const Var &v : vars_)
            if (v.record) recsize_ = v.rowElems * (uint64_t)type_size(v.type);
    // every variable must lie inside the file
    for (const Var &v : vars_) {
        uint64_t rowBytes = v.rowElems * (uint64_t)type_size(v.type);
        uint64_t last = v.rows ? (v.record ? v.begin + (v.rows - 1) * recsize_ + rowBytes : v.begin + v.rows * rowBytes) : v.begin;
        if (last > size_) {
            std::string name = v.name;
            close();
            return "Could not read '" + path + "': variable '" + name + "' reaches beyond the end of the file";
        }
    }
    return std::string();
}

bool NcFile::hasDim(const char *name) const { return dim(name, nullptr); }

bool NcFile::dim(const char *name, uint64_t *len) const {
    for (const Dim &d : dims_)
        if (d.name == name) {
            if (len) *len = d.len;
            return true;
        }
    return false;
}

const NcFile::Var *NcFile::var(const char *name) const {
    for (const Var &v : vars_)
        if (v.name == name) return &v;
    return nullptr;
}

const unsigned char *NcFile::rowPtr(const Var &v, uint64_t row) const {
    uint64_t rowBytes = v.rowElems * (uint64_t)type_size(v.type);
    return map_ + v.begin + row * (v.record ? recsize_ : rowBytes);
}

bool NcFile::readFloatRows(const Var &v, uint64_t row0, uint64_t nrows, float *dst) const {
    if (!map_ || v.type == NC_CHAR || row0 + nrows > v.rows) return false;
    const int ts = type_size(v.type);
    for (uint64_t r = 0; r < nrows; ++r) {
        const unsigned char *p = rowPtr(v, row0 + r);
        float *d = dst + r * v.rowElems;
        if (v.type == NC_FLOAT) {
            for (uint64_t e = 0; e < v.rowElems; ++e) {
                uint32_t u;
                memcpy(&u, p + 4 * e, 4);
                u = __builtin_bswap32(u);
                memcpy(d + e, &u, 4);
            }
        } else {
            for (uint64_t e = 0; e < v.rowElems; ++e) d[e] = convert<float>(p + e * ts, v.type);
        }
    }
    return true;
}

bool NcFile::readIntRows(const Var &v, uint64_t row0, uint64_t nrows, int *dst) const {
    if (!map_ || v.type == NC_CHAR || row0 + nrows > v.rows) return false;
    const int ts = type_size(v.type);
    for (uint64_t r = 0; r < nrows; ++r) {
        const unsigned char *p = rowPtr(v, row0 + r);
        for (uint64_t e = 0; e < v.rowElems; ++e) dst[r * v.rowElems + e] = convert<int>(p + e * ts, v.type);
    }
    return true;
}

bool NcFile::readTextRow(const Var &v, uint64_t row, std::string *out) const {
    if (!map_ || (v.type != NC_CHAR && v.type != NC_BYTE) || row >= v.rows) return false;
    const char *p = (const char *)rowPtr(v, row);
    size_t n = 0;
    while (n < v.rowElems && p[n]) ++n;
    out->assign(p, n);
    return true;
}

}  // namespace b2
