// Weight files of the host-side API mirror: DataReader / Initializer (Tensor/DataReader.cpp, Tensor/Initializer.cpp:21-188)
// and Net::load_weight (Tensor/Net.cpp:538-607). With these a quantized ncnn model (graph converted to .otter, parameters in
// the ncnn .bin) loads the way it does in the reference: Net::load_otter(path, CompileMode::Inference) + load_weight(bin, Ncnn).
#include <cstring>

#include "otter_api.hpp"

namespace otter {

size_t DataReaderFromStdio::read(void* buf, size_t size) const { return fread(buf, 1, size, file_); }

size_t DataReaderFromStdio::remain() const {
    const long at = ftell(file_);
    fseek(file_, 0, SEEK_END);
    const long end = ftell(file_);
    fseek(file_, at, SEEK_SET);
    return at < 0 || end < at ? 0 : (size_t)(end - at);
}

namespace {
int64_t count(const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
}
Tensor read_f32(const DataReader& dr, const std::vector<int64_t>& shape) {
    Tensor t = empty(shape, ScalarType::Float);
    const size_t bytes = (size_t)count(shape) * sizeof(float);
    if (dr.read(t.raw_data(), bytes) != bytes) {
        fprintf(stderr, "Load weight fail!\n");
        return Tensor();
    }
    return t;
}
}  // namespace

Tensor InitializerFromDataReader::load(std::vector<int64_t> shape, int /*type*/) const { return read_f32(dr_, shape); }

Tensor InitializerNcnnFromDataReader::load(std::vector<int64_t> shape, int type) const {
    if (type == 1) return read_f32(dr_, shape);
    if (type != 0) return Tensor();
    unsigned char f[4];
    if (dr_.read(f, 4) != 4) {
        fprintf(stderr, "ModelBin read flag_struct failed\n");
        return Tensor();
    }
    const unsigned int tag = (unsigned)f[0] | ((unsigned)f[1] << 8) | ((unsigned)f[2] << 16) | ((unsigned)f[3] << 24);
    const int64_t size = count(shape);
    if (tag == 0x000D4B38u) {  // int8 values, stored padded to a multiple of 4 bytes
        const size_t padded = ((size_t)size + 3) & ~(size_t)3;
        std::vector<signed char> buf(padded);
        if (dr_.read(buf.data(), padded) != padded) {
            fprintf(stderr, "ModelBin read int8_weights failed\n");
            return Tensor();
        }
        Tensor t = empty(shape, ScalarType::Byte);
        std::memcpy(t.raw_data(), buf.data(), (size_t)size);
        return t;
    }
    if (tag == 0x0002C056u) return read_f32(dr_, shape);  // raw fp32 with a tag
    const unsigned flag = (unsigned)f[0] + f[1] + f[2] + f[3];
    if (tag == 0x01306B47u || flag != 0) {
        fprintf(stderr, "ModelBin: half-precision / table-coded weights belong to fp32 layers, which this build does not run\n");
        return Tensor();
    }
    return read_f32(dr_, shape);  // tag 0: raw fp32
}

int Net::load_weight(const char* weight_path, WeightType type) {
    FILE* fp = fopen(weight_path, "rb");
    if (!fp) {
        error_ = std::string("Open weight file fail: ") + weight_path;
        return -1;
    }
    DataReaderFromStdio dr(fp);
    const int status = load_weight(dr, type);
    fclose(fp);
    return status;
}

int Net::load_weight(const DataReader& dr, WeightType type) {
    if (layers_.empty()) { error_ = "[Net] Empty graph!"; return -1; }
    if (type == WeightType::Ncnn) {
        InitializerNcnnFromDataReader initializer(dr);
        const int ret = load_weight(initializer);
        if (ret != 0) return ret;
        const size_t remain = dr.remain();
        if (remain) { error_ = "Network may initialize fail, remain weight " + std::to_string(remain); return -1; }
        return 0;
    }
    int version[2];  // Net::checkVerison (Tensor/Net.cpp:507-516): two ints in front of the reference's own files
    if (dr.read(version, sizeof(version)) != sizeof(version)) { error_ = "weight file too short"; return -1; }
    InitializerFromDataReader initializer(dr);
    return load_weight(initializer);
}

int Net::load_weight(const Initializer& initializer) {
    for (size_t i = 0; i < layers_.size(); ++i) {
        if (!layers_[i]) { error_ = "[Net] Load weight error at layer " + std::to_string(i) + ", please check the network topology."; return -1; }
        if (layers_[i]->load_model(initializer) != 0) { error_ = "[Net] layer " + std::to_string(i) + " " + layers_[i]->name + " load weight fail!"; return -1; }
    }
    if (!option.gpu) { error_ = "load_weight before compile / load_otter"; return -1; }
    for (Layer* l : layers_) {
        if (l->type() != "Convolution") { l->create_pipeline(option); continue; }
        const int rc = l->create_pipeline(option);
        if (rc != 0) { error_ = "create_pipeline of " + l->name + " failed: " + ott_last_error(option.gpu); return rc; }
    }
    return plan_fusions();
}

}  // namespace otter
