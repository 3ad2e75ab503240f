// vfold_const.hpp — C++ host-side mirror of the reference's Const dialect builder API over the C ABI of
// libvfold.so. Header-only; needs only vfold.h and the shared library.
//
// What it mirrors (reference paths are relative to src/vpux_compiler):
//   vfold::Const::ContentSetup  = Const::ContentSetup   (include/vpux/compiler/dialect/const/attributes/content.hpp:103-134;
//                                  insertion rules src/dialect/const/attributes/content.cpp:530-588)
//   vfold::Const::ContentAttr   = Const::ContentAttr    (base content + transformation list, fold())
//   vfold::Const::Content       = Const::Content        (include/vpux/compiler/dialect/const/utils/content.hpp:
//                                  getType / isSplat / getValues<T> / getSplatValue<T> / copyTo)
//   vfold::Exception            = what a VPUX_THROW on this path surfaces as; carries the vf_status
// Method names, argument meaning and failure conditions follow the reference, so a test written against the
// reference's API (tests/unit/vpux_compiler/dialect/const/) reads the same here. The data path is the GPU
// library: fold() uploads the base content, runs the transformation list on the device and materialises the
// result in the final logical element type (fold() + copyTo()).
#ifndef VFOLD_CONST_HPP_
#define VFOLD_CONST_HPP_

#include <cmath>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "vfold.h"

namespace vfold {

class Exception : public std::runtime_error {
public:
    Exception(int status, const std::string& msg): std::runtime_error(msg), _status(status) {
    }
    int status() const {
        return _status;
    }

private:
    int _status;
};

namespace details {
inline void check(int status, const char* err) {
    if (status != VF_OK) throw Exception(status, std::string(vf_status_string(status)) + ": " + err);
}
inline float halfToFloat(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            uint32_t m = man;
            do {
                ++e;
                m <<= 1;
            } while (!(m & 0x400u));
            u = sign | uint32_t(127 - 15 - e) << 23 | (m & 0x3FFu) << 13;
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | man << 13;
    } else {
        u = sign | (exp + 112) << 23 | man << 13;
    }
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline int dtypeBits(int dt) {
    switch (dt) {
    case VF_DT_F64: case VF_DT_I64: case VF_DT_U64: return 64;
    case VF_DT_F32: case VF_DT_I32: case VF_DT_U32: return 32;
    case VF_DT_F16: case VF_DT_BF16: case VF_DT_I16: case VF_DT_U16: return 16;
    case VF_DT_I8: case VF_DT_U8: return 8;
    case VF_DT_I4: case VF_DT_U4: return 4;
    case VF_DT_I1: return 1;
    default: return 0;
    }
}
}  // namespace details

// ---------------------------------------------------------------------------------------------------------
// types
// ---------------------------------------------------------------------------------------------------------
// Element type: a builtin type, !quant.uniform<...> or per-axis !quant.uniform<...>. Owns its parameters.
class ElemType {
public:
    ElemType() = default;
    /*implicit*/ ElemType(vf_dtype dt): _dtype(dt) {
    }
    static ElemType uniform(vf_dtype storage, vf_dtype expressed, double scale, int64_t zeroPoint, int64_t qmin,
                            int64_t qmax) {
        ElemType e(storage);
        e._kind = VF_ELEM_QUANT_UNIFORM;
        e._expressed = expressed;
        e._qmin = qmin;
        e._qmax = qmax;
        e._scales = {scale};
        e._zps = {zeroPoint};
        return e;
    }
    static ElemType perAxis(vf_dtype storage, vf_dtype expressed, std::vector<double> scales, std::vector<int64_t> zeroPoints,
                            int32_t axis, int64_t qmin, int64_t qmax) {
        if (scales.size() != zeroPoints.size()) throw Exception(VF_ERR_SHAPE, "scales and zero points differ in size");
        ElemType e(storage);
        e._kind = VF_ELEM_QUANT_PER_AXIS;
        e._expressed = expressed;
        e._axis = axis;
        e._qmin = qmin;
        e._qmax = qmax;
        e._scales = std::move(scales);
        e._zps = std::move(zeroPoints);
        return e;
    }
    static ElemType fromPod(const vf_elem_type& p) {
        ElemType e(static_cast<vf_dtype>(p.dtype));
        e._kind = p.kind;
        e._expressed = p.expressed;
        e._axis = p.axis;
        e._qmin = p.qmin;
        e._qmax = p.qmax;
        if (p.kind != VF_ELEM_PLAIN && p.scales && p.zps) {
            e._scales.assign(p.scales, p.scales + p.nparams);
            e._zps.assign(p.zps, p.zps + p.nparams);
        }
        return e;
    }
    vf_elem_type pod() const {  // borrows this object's parameter arrays
        vf_elem_type p{};
        p.kind = _kind;
        p.dtype = _dtype;
        p.expressed = _expressed;
        p.axis = _axis;
        p.qmin = _qmin;
        p.qmax = _qmax;
        p.nparams = int64_t(_scales.size());
        p.scales = _scales.empty() ? nullptr : _scales.data();
        p.zps = _zps.empty() ? nullptr : _zps.data();
        return p;
    }
    bool isQuantized() const {
        return _kind != VF_ELEM_PLAIN;
    }
    int32_t kind() const {
        return _kind;
    }
    vf_dtype dtype() const {
        return static_cast<vf_dtype>(_dtype);
    }
    vf_dtype expressed() const {
        return static_cast<vf_dtype>(_expressed);
    }
    int32_t axis() const {
        return _axis;
    }
    int64_t qmin() const {
        return _qmin;
    }
    int64_t qmax() const {
        return _qmax;
    }
    const std::vector<double>& scales() const {
        return _scales;
    }
    const std::vector<int64_t>& zeroPoints() const {
        return _zps;
    }
    bool operator==(const ElemType& o) const {
        return _kind == o._kind && _dtype == o._dtype && _expressed == o._expressed && _axis == o._axis && _qmin == o._qmin &&
               _qmax == o._qmax && _scales == o._scales && _zps == o._zps;
    }

private:
    int32_t _kind = VF_ELEM_PLAIN;
    int32_t _dtype = VF_DT_INVALID;
    int32_t _expressed = VF_DT_INVALID;
    int32_t _axis = -1;
    int64_t _qmin = 0, _qmax = 0;
    std::vector<double> _scales;
    std::vector<int64_t> _zps;
};

// Ranked tensor type: logical shape, element type, DimsOrder code (0 = identity).
class TensorType {
public:
    TensorType() = default;
    TensorType(std::vector<int64_t> shape, ElemType elem, vf_dims_order order = 0)
            : _shape(std::move(shape)), _elem(std::move(elem)), _order(order) {
        if (_shape.size() > VF_MAX_RANK) throw Exception(VF_ERR_INVALID_ARG, "rank above VF_MAX_RANK");
    }
    static TensorType fromPod(const vf_tensor_type& p) {
        return TensorType(std::vector<int64_t>(p.shape, p.shape + p.rank), ElemType::fromPod(p.elem), p.order);
    }
    vf_tensor_type pod() const {  // borrows the element type's parameter arrays
        vf_tensor_type p{};
        p.elem = _elem.pod();
        p.rank = int32_t(_shape.size());
        p.order = _order;
        for (size_t i = 0; i < _shape.size(); ++i) p.shape[i] = _shape[i];
        return p;
    }
    const std::vector<int64_t>& getShape() const {
        return _shape;
    }
    const ElemType& getElementType() const {
        return _elem;
    }
    vf_dims_order getDimsOrder() const {
        return _order;
    }
    int64_t getNumElements() const {
        int64_t n = 1;
        for (int64_t s : _shape) n *= s;
        return n;
    }

private:
    std::vector<int64_t> _shape;
    ElemType _elem;
    vf_dims_order _order = 0;
};

// ---------------------------------------------------------------------------------------------------------
// device context (one GPU, one stream); the reference has no counterpart — folding there runs on the host
// ---------------------------------------------------------------------------------------------------------
class Context {
public:
    explicit Context(int device = 0, const vf_options* opts = nullptr, void* externalStream = nullptr) {
        char err[512] = {0};
        details::check(vf_ctx_create(device, opts, externalStream, &_ctx, err, sizeof(err)), err);
    }
    ~Context() {
        vf_ctx_destroy(_ctx);
    }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
    vf_ctx* get() const {
        return _ctx;
    }
    // Waits for the context's stream; with VF_OPT_ASYNC this is also where deferred kernel-side failures surface.
    void synchronize() const {
        char err[512] = {0};
        details::check(vf_ctx_synchronize(_ctx, err, sizeof(err)), err);
    }

private:
    vf_ctx* _ctx = nullptr;
};

namespace Const {

// ---------------------------------------------------------------------------------------------------------
// Const::Content: the folded constant, materialised in its final logical element type
// ---------------------------------------------------------------------------------------------------------
class Content {
public:
    Content(TensorType type, bool isSplat, std::vector<uint8_t> data): _type(std::move(type)), _splat(isSplat), _data(std::move(data)) {
    }
    const TensorType& getType() const {
        return _type;
    }
    bool isSplat() const {
        return _splat;
    }
    // bytes as copyTo() lays them out (sub-byte types packed, low bits first)
    const std::vector<uint8_t>& getRawStorageBuf() const {
        return _data;
    }
    void copyTo(void* dst, size_t dstBytes) const {
        if (dstBytes < _data.size()) throw Exception(VF_ERR_BUFFER_TOO_SMALL, "Byte sizes of the input buffer and stored elements are different");
        std::memcpy(dst, _data.data(), _data.size());
    }
    // Elements converted to T (reference: Content::getValues<T>() converts the stored elements on access).
    template <typename T>
    std::vector<T> getValues() const {
        const int dt = _type.getElementType().dtype();
        const int bits = details::dtypeBits(dt);
        if (bits == 0) throw Exception(VF_ERR_UNSUPPORTED, "unknown element type");
        const size_t n = bits >= 8 ? _data.size() / size_t(bits / 8) : _data.size() * size_t(8 / bits);
        std::vector<T> out(n);
        for (size_t i = 0; i < n; ++i) out[i] = elementAs<T>(dt, bits, i);
        return out;
    }
    template <typename T>
    T getSplatValue() const {
        if (!_splat) throw Exception(VF_ERR_SPLAT, "Expected the attribute to be a splat value");
        return getValues<T>().at(0);
    }

private:
    template <typename T>
    T elementAs(int dt, int bits, size_t i) const {
        const uint8_t* p = _data.data();
        switch (dt) {
        case VF_DT_F32: { float v; std::memcpy(&v, p + 4 * i, 4); return static_cast<T>(v); }
        case VF_DT_F64: { double v; std::memcpy(&v, p + 8 * i, 8); return static_cast<T>(v); }
        case VF_DT_F16: { uint16_t v; std::memcpy(&v, p + 2 * i, 2); return static_cast<T>(details::halfToFloat(v)); }
        case VF_DT_BF16: {
            uint16_t v;
            std::memcpy(&v, p + 2 * i, 2);
            const uint32_t u = uint32_t(v) << 16;
            float f;
            std::memcpy(&f, &u, 4);
            return static_cast<T>(f);
        }
        case VF_DT_I8: return static_cast<T>(static_cast<int8_t>(p[i]));
        case VF_DT_U8: return static_cast<T>(p[i]);
        case VF_DT_I16: { int16_t v; std::memcpy(&v, p + 2 * i, 2); return static_cast<T>(v); }
        case VF_DT_U16: { uint16_t v; std::memcpy(&v, p + 2 * i, 2); return static_cast<T>(v); }
        case VF_DT_I32: { int32_t v; std::memcpy(&v, p + 4 * i, 4); return static_cast<T>(v); }
        case VF_DT_U32: { uint32_t v; std::memcpy(&v, p + 4 * i, 4); return static_cast<T>(v); }
        case VF_DT_I64: { int64_t v; std::memcpy(&v, p + 8 * i, 8); return static_cast<T>(v); }
        case VF_DT_U64: { uint64_t v; std::memcpy(&v, p + 8 * i, 8); return static_cast<T>(v); }
        default: {  // sub-byte: element i sits in the low bits first
            const int per = 8 / bits;
            const unsigned raw = (p[i / per] >> (bits * int(i % per))) & ((1u << bits) - 1u);
            if (dt == VF_DT_I4) return static_cast<T>(raw >= 8 ? int(raw) - 16 : int(raw));
            return static_cast<T>(raw);
        }
        }
    }

    TensorType _type;
    bool _splat;
    std::vector<uint8_t> _data;
};

class ContentAttr;
class Content;

// ---------------------------------------------------------------------------------------------------------
// Const::ContentSetup: collects the transformation list. Every builder returns a new setup (the reference
// moves *this into the result); transformations are inserted by their position requirement: BitPack must be
// LAST, Sparsify / GetSparsityMap PREFERRED_LAST (attr_interfaces.hpp:24-28, content.cpp:530-588).
// ---------------------------------------------------------------------------------------------------------
class ContentSetup {
public:
    explicit ContentSetup(TensorType baseType): _baseType(std::move(baseType)) {
    }
    const TensorType& getBaseType() const {
        return _baseType;
    }
    size_t size() const {
        return _items.size();
    }
    // kinds of the collected transformations in application order
    std::vector<int> getTransformationKinds() const {
        std::vector<int> k;
        for (const auto& it : _items) k.push_back(it->t.kind);
        return k;
    }

    ContentSetup castElemType(const ElemType& e) const { return withElem(VF_T_CAST_ELEM_TYPE, e); }
    ContentSetup convertElemType(const ElemType& e) const { return withElem(VF_T_CONVERT_ELEM_TYPE, e); }
    ContentSetup quantize(const ElemType& e) const { return withElem(VF_T_QUANTIZE, e); }
    ContentSetup dequantize() const { return append(make(VF_T_DEQUANTIZE)); }
    ContentSetup rescale(double scale) const {
        auto it = make(VF_T_RESCALE);
        it->t.value = scale;
        return append(std::move(it));
    }
    ContentSetup add(double bias) const {
        auto it = make(VF_T_ADD);
        it->t.value = bias;
        return append(std::move(it));
    }
    ContentSetup reshape(const std::vector<int64_t>& shape) const {
        auto it = make(VF_T_RESHAPE);
        fill(it->t.a, it->t.rank, shape);
        return append(std::move(it));
    }
    ContentSetup reorder(vf_dims_order order) const { return withOrder(VF_T_REORDER, order); }
    ContentSetup transpose(vf_dims_order order) const { return withOrder(VF_T_TRANSPOSE, order); }
    ContentSetup layoutCast(vf_dims_order order) const { return withOrder(VF_T_LAYOUT_CAST, order); }
    ContentSetup memPermute(vf_dims_order dstOrder, vf_dims_order memPerm) const {
        auto it = make(VF_T_MEM_PERMUTE);
        it->t.order = dstOrder;
        it->t.mem_perm = memPerm;
        return append(std::move(it));
    }
    ContentSetup padWithZero(const std::vector<int64_t>& padBefore, const std::vector<int64_t>& padAfter) const {
        if (padBefore.size() != padAfter.size())
            throw Exception(VF_ERR_SHAPE, "Got non consistent 'padBefore' and 'padAfter' values in 'PadWithZeroAttr'");
        auto it = make(VF_T_PAD_WITH_ZERO);
        fill(it->t.a, it->t.rank, padBefore);
        fill(it->t.b, it->t.rank, padAfter);
        return append(std::move(it));
    }
    ContentSetup subview(const std::vector<int64_t>& offset, const std::vector<int64_t>& shape) const {
        if (offset.size() != shape.size()) throw Exception(VF_ERR_SHAPE, "Got inconsistent 'offset' and 'shape' values in 'SubViewAttr'");
        auto it = make(VF_T_SUBVIEW);
        fill(it->t.a, it->t.rank, offset);
        fill(it->t.b, it->t.rank, shape);
        return append(std::move(it));
    }
    ContentSetup bitPack(int32_t width) const {
        auto it = make(VF_T_BIT_PACK);
        it->t.width = width;
        return append(std::move(it));
    }
    ContentSetup swizzleConstant(uint64_t swizzleKey, uint64_t arch) const {
        auto it = make(VF_T_SWIZZLE_CONSTANT);
        it->t.rank = 2;
        it->t.a[0] = int64_t(swizzleKey);
        it->t.a[1] = int64_t(arch);
        return append(std::move(it));
    }
    // VPUIP::SparsityCompressionAttr as RelocateWeightsTable reads it (alignment 0 = the 16-byte default)
    struct SparsityCompression {
        int64_t axis = 0;
        std::vector<int64_t> numElems;
        int64_t alignment = 0;
    };
    // content_setup.cpp:82-92
    ContentSetup relocateWeightsTablePointers(const std::vector<uint32_t>& weightsPtr, uint64_t sparsityPtr,
                                              const std::vector<int64_t>& offsets, uint64_t weightsTableSize,
                                              uint64_t weightsElemBitSize = 0, const SparsityCompression* weightsCompression = nullptr,
                                              uint64_t channelOffset = 0) const {
        if (weightsPtr.size() != offsets.size() || offsets.empty() || offsets.size() > VF_MAX_CLUSTERS)
            throw Exception(VF_ERR_INVALID_ARG, "weightsPtr and offsets need one entry per cluster");
        auto it = make(VF_T_RELOCATE_WEIGHTS_TABLE);
        vf_relocate& r = it->t.relocate;
        r.n_clusters = int32_t(offsets.size());
        r.sparsity_ptr = int32_t(sparsityPtr);
        for (size_t i = 0; i < offsets.size(); ++i) {
            r.weights_ptr[i] = int32_t(weightsPtr[i]);
            r.offsets[i] = offsets[i];
        }
        r.weights_table_size = int64_t(weightsTableSize);
        r.weights_elem_bit_size = int64_t(weightsElemBitSize);
        r.channel_offset = int64_t(channelOffset);
        if (weightsCompression) {
            it->numElems = weightsCompression->numElems;
            it->hasCompression = true;
            r.compression_axis = weightsCompression->axis;
            r.alignment = weightsCompression->alignment;
        }
        return append(std::move(it));
    }
    ContentSetup reverse(int64_t axis) const {
        auto it = make(VF_T_REVERSE);
        it->t.rank = 1;
        it->t.a[0] = axis;
        return append(std::move(it));
    }
    ContentSetup broadcast(int64_t axis, int64_t value) const {
        auto it = make(VF_T_BROADCAST);
        it->t.rank = 2;
        it->t.a[0] = axis;
        it->t.a[1] = value;
        return append(std::move(it));
    }
    ContentSetup expandDilated(const std::vector<int64_t>& dilations) const {
        if (dilations.size() != 2) throw Exception(VF_ERR_INVALID_ARG, "ExpandDilated takes the Y and X dilations");
        auto it = make(VF_T_EXPAND_DILATED);
        it->t.rank = 2;
        it->t.a[0] = dilations[0];
        it->t.a[1] = dilations[1];
        return append(std::move(it));
    }
    ContentSetup scalarMultInverse() const { return append(make(VF_T_SCALAR_MULT_INVERSE)); }
    ContentSetup changeShapeAndElemType(const std::vector<int64_t>& shape, const ElemType& e) const {
        auto it = make(VF_T_CHANGE_SHAPE_AND_ELEM_TYPE);
        fill(it->t.a, it->t.rank, shape);
        it->elem = e;
        return append(std::move(it));
    }
    ContentSetup getSparsityMap() const { return append(make(VF_T_GET_SPARSITY_MAP)); }
    ContentSetup sparsify(bool compressOutputType, const std::vector<int64_t>& numActualElements = {}) const {
        auto it = make(VF_T_SPARSIFY);
        it->t.compress_output = compressOutputType ? 1 : 0;
        for (int64_t v : numActualElements)
            if (v < 0) throw Exception(VF_ERR_INVALID_ARG, "Got negative elem number value in 'numActualElements' for 'SparsifyAttr'");
        it->counts = numActualElements;
        return append(std::move(it));
    }

    // The list after the rewriting the reference performs on every insertion (content.cpp:530-588): consecutive
    // transformations fused, no-op reorders dropped, SubView / Reshape moved towards the front. The builders
    // above keep the list as given; this returns the list the reference's ContentSetup would hold.
    ContentSetup optimize() const {
        const vf_tensor_type base = _baseType.pod();
        const std::vector<vf_transform> in = pods();
        std::vector<vf_transform> out(in.size() + 1);
        std::vector<double> sb(1 << 16);
        std::vector<int64_t> zb(1 << 16);
        int n = 0;
        char err[512] = {0};
        details::check(vf_optimize_transforms(&base, in.data(), int(in.size()), out.data(), int(out.size()), &n, sb.data(), zb.data(),
                                              int64_t(sb.size()), err, sizeof(err)),
                       err);
        ContentSetup res(_baseType);
        for (int i = 0; i < n; ++i) {
            auto it = std::make_shared<Item>();
            it->t = out[size_t(i)];
            const int k = it->t.kind;
            if (k == VF_T_CAST_ELEM_TYPE || k == VF_T_CONVERT_ELEM_TYPE || k == VF_T_QUANTIZE || k == VF_T_CHANGE_SHAPE_AND_ELEM_TYPE)
                it->elem = ElemType::fromPod(it->t.elem);
            if (it->t.num_actual) it->counts.assign(it->t.num_actual, it->t.num_actual + it->t.n_num_actual);
            if (k == VF_T_RELOCATE_WEIGHTS_TABLE && it->t.relocate.num_elems) {
                it->numElems.assign(it->t.relocate.num_elems, it->t.relocate.num_elems + it->t.relocate.n_num_elems);
                it->hasCompression = true;
            }
            res._items.push_back(std::move(it));
        }
        return res;
    }
    // parameters of transformation i (for checks in tests)
    vf_transform at(size_t i) const {
        return pods().at(i);
    }

    // = ContentSetup::get(): the attribute over `base` (bytes in `storage`, borrowed until fold() returns)
    inline ContentAttr get(const void* base, size_t baseBytes, bool isSplat = false, vf_dtype storage = VF_DT_INVALID) const;

    // the POD list handed to the C ABI; valid while this setup lives
    std::vector<vf_transform> pods() const {
        std::vector<vf_transform> v;
        for (const auto& it : _items) {
            vf_transform t = it->t;
            t.elem = it->elem.pod();
            t.num_actual = it->counts.empty() ? nullptr : it->counts.data();
            t.n_num_actual = int64_t(it->counts.size());
            static const int64_t kNone = 0;  // an empty numElems list is still "compressed"
            t.relocate.num_elems = !it->hasCompression ? nullptr : it->numElems.empty() ? &kNone : it->numElems.data();
            t.relocate.n_num_elems = it->hasCompression ? int64_t(it->numElems.size()) : 0;
            v.push_back(t);
        }
        return v;
    }

private:
    struct Item {
        vf_transform t{};
        ElemType elem;
        std::vector<int64_t> counts;
        std::vector<int64_t> numElems;  // RelocateWeightsTable weightsCompression
        bool hasCompression = false;
    };
    static int position(int kind) {  // 0 = NONE, 1 = PREFERRED_LAST, 2 = LAST
        if (kind == VF_T_BIT_PACK || kind == VF_T_SWIZZLE_CONSTANT) return 2;
        if (kind == VF_T_SPARSIFY || kind == VF_T_GET_SPARSITY_MAP) return 1;
        return 0;
    }
    static std::shared_ptr<Item> make(int kind) {
        auto it = std::make_shared<Item>();
        it->t.kind = kind;
        return it;
    }
    static void fill(int64_t* dst, int32_t& rank, const std::vector<int64_t>& v) {
        if (v.size() > VF_MAX_RANK) throw Exception(VF_ERR_INVALID_ARG, "rank above VF_MAX_RANK");
        rank = int32_t(v.size());
        for (size_t i = 0; i < v.size(); ++i) dst[i] = v[i];
    }
    ContentSetup withElem(int kind, const ElemType& e) const {
        auto it = make(kind);
        it->elem = e;
        return append(std::move(it));
    }
    ContentSetup withOrder(int kind, vf_dims_order order) const {
        auto it = make(kind);
        it->t.order = order;
        return append(std::move(it));
    }
    ContentSetup append(std::shared_ptr<Item> it) const {
        ContentSetup out(*this);
        // upper bound on the position requirement keeps [NONE..., PREFERRED_LAST..., LAST...] stable
        size_t pos = out._items.size();
        for (size_t i = 0; i < out._items.size(); ++i) {
            if (position(out._items[i]->t.kind) > position(it->t.kind)) {
                pos = i;
                break;
            }
        }
        out._items.insert(out._items.begin() + long(pos), std::move(it));
        const size_t n = out._items.size();
        if (n >= 2 && position(out._items[n - 2]->t.kind) == 2) throw Exception(VF_ERR_POSITION, "At most 1 attribute with LAST requirement allowed!");
        return out;
    }

    TensorType _baseType;
    std::vector<std::shared_ptr<Item>> _items;
};

// ---------------------------------------------------------------------------------------------------------
// Const::ContentAttr: base content + transformation list
// ---------------------------------------------------------------------------------------------------------
class ContentAttr {
public:
    ContentAttr(ContentSetup setup, const void* base, size_t baseBytes, bool isSplat, vf_dtype storage)
            : _setup(std::move(setup)), _base(base), _baseBytes(baseBytes), _splat(isSplat), _storage(storage) {
        if (_storage == VF_DT_INVALID) _storage = _setup.getBaseType().getElementType().dtype();
    }
    // further transformations on top of this attribute (reference: ContentAttr::transform())
    const ContentSetup& transform() const {
        return _setup;
    }
    // = ContentAttr::getType(): the type after all transformations (inferFinalTypeAndSplat, content.cpp:519-528)
    TensorType getType() const {
        bool splat;
        uint64_t bytes;
        return infer(splat, bytes);
    }
    bool isSplat() const {
        bool splat;
        uint64_t bytes;
        infer(splat, bytes);
        return splat;
    }
    // = fold() + copyTo(): applies the list on the GPU and returns the materialised content. `dstBytes`
    // overrides the destination size (Sparsify<false> writes fewer bytes than the inferred type holds).
    Content fold(const Context& ctx, uint64_t dstBytes = 0, vf_stats* stats = nullptr) const {
        bool splat;
        uint64_t need;
        infer(splat, need);
        const TensorType& bt = _setup.getBaseType();
        vf_content c{};
        c.type = bt.pod();
        c.storage_dtype = _storage;
        c.is_splat = _splat ? 1 : 0;
        c.mem_kind = VF_MEM_HOST;
        c.data = _base;
        c.nbytes = _baseBytes;
        const std::vector<vf_transform> t = _setup.pods();
        std::vector<uint8_t> dst(size_t(dstBytes ? dstBytes : need));
        if (dst.empty()) dst.resize(1);
        uint64_t written = 0;
        vf_tensor_type outPod{};
        std::vector<double> sb(kParamsCap);
        std::vector<int64_t> zb(kParamsCap);
        char err[512] = {0};
        details::check(vf_fold(ctx.get(), &c, t.data(), int(t.size()), dst.data(), dstBytes ? dstBytes : need, VF_MEM_HOST, &written,
                               &outPod, sb.data(), zb.data(), kParamsCap, stats, err, sizeof(err)),
                       err);
        dst.resize(size_t(written));
        return Content(TensorType::fromPod(outPod), splat, std::move(dst));
    }

    // the POD view of the base content (borrowing this attribute's buffer)
    vf_content basePod() const {
        vf_content c{};
        c.type = _setup.getBaseType().pod();
        c.storage_dtype = _storage;
        c.is_splat = _splat ? 1 : 0;
        c.mem_kind = VF_MEM_HOST;
        c.data = _base;
        c.nbytes = _baseBytes;
        return c;
    }

private:
    friend class BackgroundConstantFolding;
    friend std::vector<Content> foldConstants(const Context&, const std::vector<ContentAttr>&, uint64_t, uint64_t, vf_fold_batch_stats*,
                                              std::vector<int>*);
    static constexpr int64_t kParamsCap = 1 << 16;
    TensorType infer(bool& splat, uint64_t& bytes) const {
        const vf_tensor_type base = _setup.getBaseType().pod();
        const std::vector<vf_transform> t = _setup.pods();
        vf_tensor_type out{};
        int outSplat = 0;
        std::vector<double> sb(kParamsCap);
        std::vector<int64_t> zb(kParamsCap);
        char err[512] = {0};
        details::check(vf_infer_type(&base, _splat ? 1 : 0, t.data(), int(t.size()), &out, &outSplat, sb.data(), zb.data(), kParamsCap,
                                     &bytes, err, sizeof(err)),
                       err);
        splat = outSplat != 0;
        return TensorType::fromPod(out);
    }

    ContentSetup _setup;
    const void* _base;
    size_t _baseBytes;
    bool _splat;
    vf_dtype _storage;
};

inline ContentAttr ContentSetup::get(const void* base, size_t baseBytes, bool isSplat, vf_dtype storage) const {
    return ContentAttr(*this, base, baseBytes, isSplat, storage);
}

// ---------------------------------------------------------------------------------------------------------
// Const::BackgroundConstantFolding + Const::ConstantFoldingCache (utils/constant_folding_in_background.hpp:25-72,
// utils/constant_folding_cache.hpp:130-262) over vf_folder: requests are folded by worker threads on the
// device and the folded contents are cached there; fold() is ContentAttr::fold() through that cache.
// The base buffer of a queued attribute must stay valid until waitIdle() (or the destructor) returns.
// ---------------------------------------------------------------------------------------------------------
// ConstantFoldingPass::safeRunOnFunc (const/passes/constant_folding.cpp:85-159) over a list of attributes in place
// of a function's const.Declare ops: every constant is folded into a buffer of its own with the pass's schedule.
// `threshold` / `tinyThreshold` of 0 are the pass's 300 MB / 1 KB; `groups` receives where each constant ran.
inline std::vector<Content> foldConstants(const Context& ctx, const std::vector<ContentAttr>& attrs, uint64_t threshold = 0,
                                          uint64_t tinyThreshold = 0, vf_fold_batch_stats* batchStats = nullptr,
                                          std::vector<int>* groups = nullptr) {
    const size_t n = attrs.size();
    std::vector<vf_fold_job> jobs(n);
    std::vector<std::vector<vf_transform>> lists(n);
    std::vector<std::vector<uint8_t>> dst(n);
    std::vector<TensorType> types;
    std::vector<char> splats(n);
    types.reserve(n);
    for (size_t j = 0; j < n; ++j) {
        bool splat;
        uint64_t need;
        types.push_back(attrs[j].infer(splat, need));
        splats[j] = splat;
        lists[j] = attrs[j].transform().pods();
        dst[j].resize(size_t(need ? need : 1));
        vf_fold_job& jb = jobs[j];
        jb = vf_fold_job{};
        jb.base = attrs[j].basePod();
        jb.t = lists[j].data();
        jb.n = int(lists[j].size());
        jb.dst_mem_kind = VF_MEM_HOST;
        jb.dst = dst[j].data();
        jb.dst_bytes = need;
    }
    const vf_fold_batch_options opts{threshold, tinyThreshold};
    char err[512] = {0};
    details::check(vf_fold_batch(ctx.get(), jobs.data(), int(n), &opts, batchStats, nullptr, err, sizeof(err)), err);
    std::vector<Content> out;
    out.reserve(n);
    if (groups) groups->clear();
    for (size_t j = 0; j < n; ++j) {
        dst[j].resize(size_t(jobs[j].dst_written));
        out.emplace_back(types[j], splats[j] != 0, std::move(dst[j]));
        if (groups) groups->push_back(jobs[j].group);
    }
    return out;
}

class BackgroundConstantFolding {
public:
    // memoryUsageLimit in MB as in the reference (0 = the library's default)
    BackgroundConstantFolding(int device, size_t maxConcurrentTasks, bool collectStatistics, size_t memoryUsageLimit = 0,
                              double cacheCleanThreshold = 0.8) {
        vf_folder_options o{};
        o.memory_limit_bytes = uint64_t(memoryUsageLimit) << 20;
        o.clean_threshold = cacheCleanThreshold;
        o.max_concurrent_tasks = int32_t(maxConcurrentTasks);
        o.collect_statistics = collectStatistics ? 1 : 0;
        char err[512] = {0};
        details::check(vf_folder_create(device, &o, &_folder, err, sizeof(err)), err);
    }
    ~BackgroundConstantFolding() {
        vf_folder_destroy(_folder);
    }
    BackgroundConstantFolding(const BackgroundConstantFolding&) = delete;
    BackgroundConstantFolding& operator=(const BackgroundConstantFolding&) = delete;

    // ConstantFoldingCache::enqueueRequest(FoldingRequest{attr, newTransformation}); `newIndex` = position of the
    // transformation appended last, -1 for none; `baseId` = the caller's identity of the base bytes, 0 = hash them
    void enqueueRequest(const ContentAttr& attr, int newIndex = -1, uint64_t baseId = 0) {
        const vf_content c = attr.basePod();
        const std::vector<vf_transform> t = attr.transform().pods();
        char err[512] = {0};
        details::check(vf_folder_enqueue(_folder, &c, baseId, t.data(), int(t.size()), newIndex, err, sizeof(err)), err);
    }
    void enqueueRequest(const ContentAttr& originalAttr, const ContentAttr& newAttr, uint64_t baseId = 0) {  // EquivalenceRequest
        const vf_content c = originalAttr.basePod();
        const std::vector<vf_transform> t0 = originalAttr.transform().pods(), t1 = newAttr.transform().pods();
        char err[512] = {0};
        details::check(vf_folder_enqueue_equivalence(_folder, &c, baseId, t0.data(), int(t0.size()), t1.data(), int(t1.size()), err,
                                                     sizeof(err)),
                       err);
    }
    void waitIdle() {
        char err[512] = {0};
        details::check(vf_folder_wait_idle(_folder, err, sizeof(err)), err);
    }
    bool hasContent(const ContentAttr& attr, uint64_t baseId = 0) {
        const vf_content c = attr.basePod();
        const std::vector<vf_transform> t = attr.transform().pods();
        int found = 0;
        char err[512] = {0};
        details::check(vf_folder_has_content(_folder, &c, baseId, t.data(), int(t.size()), &found, err, sizeof(err)), err);
        return found != 0;
    }
    // ContentAttr::fold() with the cache consulted first (attributes/content.cpp:371-397)
    Content fold(const ContentAttr& attr, bool* fromCache = nullptr, uint64_t baseId = 0) {
        bool splat;
        uint64_t need;
        attr.infer(splat, need);
        const vf_content c = attr.basePod();
        const std::vector<vf_transform> t = attr.transform().pods();
        std::vector<uint8_t> dst(size_t(need ? need : 1));
        uint64_t written = 0;
        vf_tensor_type outPod{};
        std::vector<double> sb(ContentAttr::kParamsCap);
        std::vector<int64_t> zb(ContentAttr::kParamsCap);
        int hit = 0;
        char err[512] = {0};
        details::check(vf_folder_fold(_folder, &c, baseId, t.data(), int(t.size()), dst.data(), need, VF_MEM_HOST, &written, &outPod,
                                      sb.data(), zb.data(), ContentAttr::kParamsCap, &hit, err, sizeof(err)),
                       err);
        if (fromCache) *fromCache = hit != 0;
        dst.resize(size_t(written));
        return Content(TensorType::fromPod(outPod), splat, std::move(dst));
    }
    vf_folder_stats getStatistics() {
        vf_folder_stats s{};
        vf_folder_statistics(_folder, &s);
        return s;
    }

private:
    vf_folder* _folder = nullptr;
};

}  // namespace Const
}  // namespace vfold

#endif  // VFOLD_CONST_HPP_
