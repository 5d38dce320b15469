// Reader for netCDF classic files (CDF-1 and CDF-2, "64-bit offset"), the on-disk format of the
// reference toolkit's data sets (CURRENNT_codes/README section 5; written by
// pyTools/dataTools/ncDataHandle.py through scipy's netcdf_file with version=2).
//
// The reference reads through libnetcdf (data_sets/DataSet.cpp:65-195: nc_inq_dimid, nc_inq_dimlen,
// nc_get_vara_{text,int,float}).  Here the file is mapped into memory and parsed directly from the
// published classic-format grammar; values are converted from big-endian straight into the caller's
// buffer, so a fraction is assembled with one pass over the bytes and no cache file.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

namespace b2 {

class NcFile {
public:
    enum Type { NC_BYTE = 1, NC_CHAR = 2, NC_SHORT = 3, NC_INT = 4, NC_FLOAT = 5, NC_DOUBLE = 6 };
    struct Dim {
        std::string name;
        uint64_t len;       // 0 in the file = the record dimension; replaced by numrecs after parsing
        bool record;
    };
    struct Var {
        std::string name;
        std::vector<int> dimids;
        int type;
        uint64_t vsize, begin;
        bool record;
        uint64_t rowElems;  // elements per index of the first dimension
        uint64_t rows;      // extent of the first dimension (1 for scalars)
    };

    NcFile() {}
    ~NcFile();
    NcFile(const NcFile &) = delete;
    NcFile &operator=(const NcFile &) = delete;

    // returns an empty string on success, else the reason
    std::string open(const std::string &path);
    void close();

    bool hasDim(const char *name) const;
    // false when the dimension does not exist
    bool dim(const char *name, uint64_t *len) const;
    const Var *var(const char *name) const;

    // rows [row0, row0 + nrows) of a variable, converted to float / int; false when out of range
    // or when the type cannot be converted (text as numbers and the like)
    bool readFloatRows(const Var &v, uint64_t row0, uint64_t nrows, float *dst) const;
    bool readIntRows(const Var &v, uint64_t row0, uint64_t nrows, int *dst) const;
    // one row of a char variable as a string (stops at the first NUL)
    bool readTextRow(const Var &v, uint64_t row, std::string *out) const;

    const std::string &path() const { return path_; }

private:
    const unsigned char *rowPtr(const Var &v, uint64_t row) const;
    std::string path_;
    const unsigned char *map_ = nullptr;
    size_t size_ = 0;
    int version_ = 0;
    uint64_t numrecs_ = 0, recsize_ = 0;
    std::vector<Dim> dims_;
    std::vector<Var> vars_;
};

}  // namespace b2
