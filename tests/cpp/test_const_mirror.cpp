// Tests of the C++ host mirror (include/vfold_const.hpp) written the way the reference's own unit tests of
// the Const dialect are (tests/unit/vpux_compiler/dialect/const/content_tests.cpp, cited as UT:lines):
// build a ContentAttr through ContentSetup, fold(), compare getValues<T>() with the expected numbers.
//
//   test_const_mirror --host   builder / type-inference / error checks that need no GPU
//   test_const_mirror          everything, folding on cuda:0
// Exit code 0 = all checks passed; every failed check prints its location.
#include <cstdio>
#include <cstring>
#include <numeric>

#include "vfold_const.hpp"

using namespace vfold;

static int g_failed = 0;
#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("%s:%d: EXPECT(%s) failed\n", __FILE__, __LINE__, #cond); \
            ++g_failed;                                                     \
        }                                                                   \
    } while (0)

template <typename T>
static std::vector<T> generateValues(size_t n) {  // UT:43-51
    std::vector<T> v(n);
    for (size_t i = 0; i < n; ++i) v[i] = static_cast<T>(i);
    return v;
}

template <typename T>
static size_t bytesOf(const std::vector<T>& v) {
    return v.size() * sizeof(T);
}

// ---- host-only ------------------------------------------------------------------------------------------
static void positionRequirement() {  // UT:1724-1749 (BitPack stands in for the LAST-positioned SwizzleConstant)
    const TensorType baseType({1, 1, 3, 3}, VF_DT_F32);
    const auto setup = Const::ContentSetup(baseType).rescale(10.0).bitPack(4).sparsify(false).castElemType(VF_DT_F16);
    const std::vector<int> expected = {VF_T_RESCALE, VF_T_CAST_ELEM_TYPE, VF_T_SPARSIFY, VF_T_BIT_PACK};
    EXPECT(setup.getTransformationKinds() == expected);
    bool thrown = false;
    try {
        (void)setup.bitPack(4);
    } catch (const Exception& e) {
        thrown = e.status() == VF_ERR_POSITION;
    }
    EXPECT(thrown);  // "At most 1 attribute with LAST requirement allowed!"
}

static void inferTypes() {
    const TensorType baseType({2, 4, 3, 3}, VF_DT_F32);
    const std::vector<float> vals(72, 1.0f);
    const auto q = ElemType::perAxis(VF_DT_I8, VF_DT_F32, {0.1, 0.2}, {0, 0}, 0, -127, 127);
    // Quantize yields the plain storage type (quantize.cpp:108-212); CastElemType re-attaches the quantized type
    const auto attr = Const::ContentSetup(baseType)
                              .quantize(q)
                              .castElemType(q)
                              .reorder(VF_ORDER_NHWC)
                              .padWithZero({0, 0, 0, 0}, {14, 12, 0, 0})
                              .get(vals.data(), bytesOf(vals));
    const TensorType t = attr.getType();
    EXPECT((t.getShape() == std::vector<int64_t>{16, 16, 3, 3}));
    EXPECT(t.getDimsOrder() == VF_ORDER_NHWC);
    EXPECT(t.getElementType().kind() == VF_ELEM_QUANT_PER_AXIS);
    EXPECT(t.getElementType().scales().size() == 16);  // padded channels extend the per-axis parameters
    EXPECT(!attr.isSplat());

    bool thrown = false;
    try {  // Dequantize on a plain type
        (void)Const::ContentSetup(baseType).dequantize().get(vals.data(), bytesOf(vals)).getType();
    } catch (const Exception& e) {
        thrown = e.status() == VF_ERR_NOT_QUANTIZED;
    }
    EXPECT(thrown);
    thrown = false;
    try {
        (void)Const::ContentSetup(baseType).padWithZero({0, 0}, {1, 1, 1});
    } catch (const Exception& e) {
        thrown = e.status() == VF_ERR_SHAPE;
    }
    EXPECT(thrown);
}

static void remainingTransformationTypes() {
    // reverse.cpp:35-44 and inverse.cpp:40-50 keep the type; getDilatedType (utils/dilated_utils.cpp:11-34);
    // broadcast.cpp:66-83 pads the type behind the axis; change_shape_and_elem_type.cpp:62-66
    const TensorType f32({2, 3, 4, 5}, VF_DT_F32);
    const std::vector<float> vals(120, 1.0f);
    EXPECT((Const::ContentSetup(f32).reverse(1).get(vals.data(), bytesOf(vals)).getType().getShape() == std::vector<int64_t>{2, 3, 4, 5}));
    EXPECT((Const::ContentSetup(f32).expandDilated({3, 2}).get(vals.data(), bytesOf(vals)).getType().getShape() ==
            std::vector<int64_t>{2, 3, 10, 9}));
    EXPECT((Const::ContentSetup(f32).broadcast(1, 6).get(vals.data(), bytesOf(vals)).getType().getShape() == std::vector<int64_t>{2, 6, 4, 5}));
    EXPECT(Const::ContentSetup(f32).scalarMultInverse().get(vals.data(), bytesOf(vals)).getType().getElementType().dtype() == VF_DT_F32);
    const auto q = ElemType::perAxis(VF_DT_U8, VF_DT_F16, {0.5, 0.5}, {127, 127}, 1, 0, 255);
    const TensorType u8({2, 1, 1, 8}, VF_DT_U8);
    const std::vector<uint8_t> bytes(16, 7);
    const TensorType changed = Const::ContentSetup(u8).changeShapeAndElemType({1, 2, 1, 8}, q).get(bytes.data(), bytesOf(bytes)).getType();
    EXPECT((changed.getShape() == std::vector<int64_t>{1, 2, 1, 8}) && changed.getElementType().kind() == VF_ELEM_QUANT_PER_AXIS);
    bool thrown = false;
    try {  // a broadcast below the current extent
        (void)Const::ContentSetup(f32).broadcast(1, 2).get(vals.data(), bytesOf(vals)).getType();
    } catch (const Exception& e) {
        thrown = e.status() == VF_ERR_SHAPE;
    }
    EXPECT(thrown);
}

static void optimizedLists() {
    // content_setup.cpp:720-747 FuseSubView
    const TensorType i8({1, 7, 5}, VF_DT_I8);
    auto fused = Const::ContentSetup(i8).subview({0, 1, 2}, {1, 6, 3}).subview({0, 1, 1}, {1, 2, 1}).optimize();
    EXPECT(fused.size() == 1);
    EXPECT(fused.at(0).kind == VF_T_SUBVIEW && fused.at(0).a[1] == 2 && fused.at(0).a[2] == 3 && fused.at(0).b[1] == 2);
    // content_setup.cpp:903-930 SwapTransposeAndSubView
    const TensorType chw({4, 8, 3}, VF_DT_I8);
    auto swapped = Const::ContentSetup(chw).transpose(0x321).subview({0, 1, 2}, {3, 2, 1}).optimize();
    EXPECT((swapped.getTransformationKinds() == std::vector<int>{VF_T_SUBVIEW, VF_T_TRANSPOSE}));
    EXPECT(swapped.at(0).a[0] == 2 && swapped.at(0).a[1] == 1 && swapped.at(0).a[2] == 0);
    EXPECT(swapped.at(0).b[0] == 1 && swapped.at(0).b[1] == 2 && swapped.at(0).b[2] == 3);
    // content_setup.cpp:1257-1294: a per-axis type is sliced together with the view
    const TensorType u8({2, 8, 3}, VF_DT_U8);
    const auto perAxis = ElemType::perAxis(VF_DT_U8, VF_DT_F32, {2.0, 0.5}, {127, 127}, 0, 0, 255);
    auto sliced = Const::ContentSetup(u8).castElemType(perAxis).subview({0, 1, 1}, {1, 2, 1}).optimize();
    EXPECT((sliced.getTransformationKinds() == std::vector<int>{VF_T_SUBVIEW, VF_T_CAST_ELEM_TYPE}));
    EXPECT(sliced.at(1).elem.nparams == 1 && sliced.at(1).elem.scales[0] == 2.0);
    // content_setup.cpp:1644-1648: a SubView of one cluster moves before RelocateWeightsTable, which keeps that
    // cluster's pointer and the slice of the compression entries
    const TensorType table({8, 1, 1, 4}, VF_DT_I32);
    Const::ContentSetup::SparsityCompression comp;
    comp.numElems = {1, 2, 3, 4, 5, 6, 7, 8};
    comp.alignment = 16;
    auto relocated = Const::ContentSetup(table)
                             .relocateWeightsTablePointers({100, 200, 300, 400}, 200, {0, 2, 4, 6}, 128, 16, &comp, 0)
                             .subview({4, 0, 0, 0}, {2, 1, 1, 4})
                             .optimize();
    EXPECT((relocated.getTransformationKinds() == std::vector<int>{VF_T_SUBVIEW, VF_T_RELOCATE_WEIGHTS_TABLE}));
    const vf_relocate r = relocated.at(1).relocate;
    EXPECT(r.n_clusters == 1 && r.weights_ptr[0] == 300 && r.offsets[0] == 0 && r.weights_table_size == 32 && r.channel_offset == 0);
    EXPECT(r.n_num_elems == 2 && r.num_elems[0] == 5 && r.num_elems[1] == 6);
}

// ---- folding on the GPU ------------------------------------------------------------------------------------
static void quantize(const Context& ctx) {  // UT:2440-2469
    const TensorType baseType({1, 16}, VF_DT_F32);
    std::vector<float> vals(16);
    for (int i = 0; i < 16; ++i) vals[i] = -2.0f + 0.25f * float(i);
    const auto q = ElemType::uniform(VF_DT_I8, VF_DT_F32, 1.0 / 127.0, 56, -127, 127);
    const auto content = Const::ContentSetup(baseType).quantize(q).get(vals.data(), bytesOf(vals)).fold(ctx);
    EXPECT(content.getType().getElementType().dtype() == VF_DT_I8);
    const std::vector<int> expected = {-127, -127, -127, -103, -71, -39, -7, 24, 56, 88, 120, 127, 127, 127, 127, 127};
    EXPECT(content.getValues<int>() == expected);
}

static void dequantize(const Context& ctx) {  // after UT:754-788, with a non-zero zero point: (v - zp) * scale
    const TensorType baseType({1, 16}, VF_DT_I8);
    std::vector<int8_t> vals(16);
    for (int i = 0; i < 16; ++i) vals[i] = int8_t(-8 + i);
    const double scale = 0.5;
    const int64_t zp = 3;
    const auto q = ElemType::uniform(VF_DT_I8, VF_DT_F32, scale, zp, -128, 127);
    const auto content = Const::ContentSetup(baseType).castElemType(q).dequantize().get(vals.data(), bytesOf(vals)).fold(ctx);
    EXPECT(content.getType().getElementType().dtype() == VF_DT_F32);
    const auto got = content.getValues<float>();
    for (int i = 0; i < 16; ++i) EXPECT(got[size_t(i)] == float((vals[size_t(i)] - zp) * scale));
}

static void reorder(const Context& ctx) {  // UT:906-939 NCHW -> NHWC
    const int64_t C = 2, H = 2, W = 2;
    const TensorType baseType({1, C, H, W}, VF_DT_F32);
    const auto vals = generateValues<float>(8);
    const auto content = Const::ContentSetup(baseType).reorder(VF_ORDER_NHWC).get(vals.data(), bytesOf(vals)).fold(ctx);
    EXPECT(content.getType().getDimsOrder() == VF_ORDER_NHWC);
    const auto got = content.getValues<float>();
    for (int64_t c = 0; c < C; ++c)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t w = 0; w < W; ++w) EXPECT(got[size_t(c + w * C + h * C * W)] == vals[size_t(w + h * W + c * W * H)]);
}

static void padWithZeroSplat(const Context& ctx) {  // UT:1013-1050: a padded splat is no longer a splat
    const TensorType baseType({1, 2, 2, 2}, VF_DT_F32);
    const float splat = 7.0f;
    const auto attr = Const::ContentSetup(baseType).padWithZero({0, 1, 0, 0}, {0, 1, 0, 0}).get(&splat, sizeof(splat), true);
    const auto content = attr.fold(ctx);
    EXPECT(!content.isSplat());
    EXPECT((content.getType().getShape() == std::vector<int64_t>{1, 4, 2, 2}));
    const auto got = content.getValues<float>();
    for (size_t i = 0; i < got.size(); ++i) EXPECT(got[i] == ((i >= 4 && i < 12) ? splat : 0.0f));
}

static void bitPack(const Context& ctx) {  // UT:1246-1274
    const TensorType baseType({1, 2, 3}, VF_DT_I8);
    const std::vector<int8_t> vals = {1, 2, 3, 4, 5, 6};
    const auto content = Const::ContentSetup(baseType).bitPack(4).get(vals.data(), bytesOf(vals)).fold(ctx);
    EXPECT(content.getType().getElementType().dtype() == VF_DT_I4);
    EXPECT((content.getRawStorageBuf() == std::vector<uint8_t>{0x21, 0x43, 0x65}));
    EXPECT((content.getValues<int>() == std::vector<int>{1, 2, 3, 4, 5, 6}));
}

static void getSparsityMap(const Context& ctx) {  // UT:1536-1569
    const TensorType baseType({1, 1, 2, 8}, VF_DT_U8);
    const std::vector<uint8_t> vals = {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 0, 11, 0, 13, 14, 15};
    const auto content = Const::ContentSetup(baseType).getSparsityMap().get(vals.data(), bytesOf(vals)).fold(ctx);
    EXPECT((content.getType().getShape() == std::vector<int64_t>{1, 1, 1, 128}));
    std::vector<uint8_t> expected(16, 0);
    expected[0] = 0xFE;
    expected[1] = 0xEB;
    EXPECT(content.getRawStorageBuf() == expected);
}

static void sparsifyQuantized(const Context& ctx) {  // UT:1681-1722 (zero point 16)
    const TensorType baseType({2, 1, 2, 8}, VF_DT_U8);
    const std::vector<uint8_t> vals = {16, 1,  2,  3,  4,  5,  6,  7,  8,  9,  16, 11, 16, 13, 14, 15,
                                       16, 16, 18, 19, 20, 16, 22, 23, 24, 25, 26, 16, 16, 29, 30, 31};
    const std::vector<uint8_t> expected = {1,  2,  3,  4,  5,  6,  7,  8,  9,  11, 13, 14, 15, 0, 0, 0,
                                           18, 19, 20, 22, 23, 24, 25, 26, 29, 30, 31, 0,  0,  0, 0, 0};
    const auto q = ElemType::uniform(VF_DT_U8, VF_DT_F32, 1.0, 16, 0, 31);
    const auto content = Const::ContentSetup(baseType).castElemType(q).sparsify(false).get(vals.data(), bytesOf(vals)).fold(ctx);
    EXPECT(content.getRawStorageBuf() == expected);
}

static void dequantizeQuantize(const Context& ctx) {  // UT:2512-2540: the chain is the identity
    const TensorType baseType({1, 16}, VF_DT_I8);
    std::vector<int8_t> vals(16);
    for (int i = 0; i < 16; ++i) vals[size_t(i)] = int8_t(-120 + 15 * i);
    const auto q = ElemType::uniform(VF_DT_I8, VF_DT_F16, 0.003, 56, -120, 120);
    const auto content = Const::ContentSetup(baseType).castElemType(q).dequantize().quantize(q).get(vals.data(), bytesOf(vals)).fold(ctx);
    const auto got = content.getValues<int>();
    for (int i = 0; i < 16; ++i) EXPECT(got[size_t(i)] == vals[size_t(i)]);
}

static void relocateWeightsTable(const Context& ctx) {  // lit const/passes/constant_folding.mlir:597-611
    const TensorType baseType({4, 1, 1, 4}, VF_DT_I32);
    const std::vector<int32_t> vals = {1, 2, 3, 3, 2, 4, 4, 4, 3, 6, 5, 5, 4, 8, 6, 6};
    const auto content = Const::ContentSetup(baseType)
                                 .relocateWeightsTablePointers({10, 20}, 5, {0, 2}, 64, 16)
                                 .get(vals.data(), bytesOf(vals))
                                 .fold(ctx);
    const std::vector<int32_t> expected = {10, 5, 3, 3, 11, 7, 4, 4, 20, 5, 5, 5, 21, 7, 6, 6};
    EXPECT(content.getValues<int32_t>() == expected);
}

static void constantFoldingPass(const Context& ctx) {  // const/passes/constant_folding.cpp:85-159
    std::vector<float> small(64), mid(64 * 1024), large(512 * 1024);
    for (size_t i = 0; i < small.size(); ++i) small[i] = float(i) * 0.5f;
    for (size_t i = 0; i < mid.size(); ++i) mid[i] = float(int(i % 255) - 127);
    for (size_t i = 0; i < large.size(); ++i) large[i] = float(int(i % 63) - 31) * 0.25f;
    std::vector<Const::ContentAttr> attrs;
    attrs.push_back(Const::ContentSetup(TensorType({64}, VF_DT_F32)).castElemType(VF_DT_F16).get(small.data(), small.size() * 4));
    attrs.push_back(Const::ContentSetup(TensorType({512, 1024}, VF_DT_F32)).castElemType(VF_DT_F16).get(large.data(), large.size() * 4));
    attrs.push_back(Const::ContentSetup(TensorType({64, 1024}, VF_DT_F32)).castElemType(VF_DT_F16).get(mid.data(), mid.size() * 4));
    attrs.push_back(Const::ContentSetup(TensorType({64, 1024}, VF_DT_F32)).add(1.0).get(mid.data(), mid.size() * 4));
    vf_fold_batch_stats stats{};
    std::vector<int> groups;
    // threshold 1 MiB: the 2 MiB constant that opens the walk is folded alone, the two 256 KiB ones share a
    // group, the small one is tiny
    const auto folded = Const::foldConstants(ctx, attrs, 1u << 20, 0, &stats, &groups);
    EXPECT(groups == (std::vector<int>{VF_GROUP_TINY, VF_GROUP_ALONE, 0, 0}));
    EXPECT(stats.tiny == 1 && stats.alone == 1 && stats.groups == 1 && stats.synchronisations == 3);
    EXPECT(stats.max_group_bytes == 2u * 64 * 1024 * 4);
    EXPECT(folded.size() == 4);
    for (size_t j = 0; j < folded.size(); ++j) {
        const auto single = attrs[j].fold(ctx);
        EXPECT(folded[j].getRawStorageBuf() == single.getRawStorageBuf());
        EXPECT(folded[j].getType().getShape() == single.getType().getShape());
    }
    EXPECT(folded[3].getValues<float>()[5] == mid[5] + 1.0f);
}

static void foldingInBackground() {  // constant_folding_in_background_tests.cpp:36-52, 88-106 and :156-196
    Const::BackgroundConstantFolding folding(0, 2, true, 3 * 1024, 0.8);
    const TensorType baseType({100}, VF_DT_F32);
    const float baseValue = 1.0f;
    auto setup = Const::ContentSetup(baseType);
    for (int i = 0; i < 5; ++i) setup = setup.add(1.0);
    const auto attr = setup.get(&baseValue, sizeof(baseValue), true);
    folding.enqueueRequest(attr);
    folding.waitIdle();
    bool fromCache = false;
    const auto content = folding.fold(attr, &fromCache);
    EXPECT(fromCache);
    EXPECT(content.getValues<float>() == std::vector<float>(100, 6.0f));
    // an equivalence request re-keys the cached result of the two SubViews to the fused one
    const auto attr1 = Const::ContentSetup(baseType).subview({0}, {50}).subview({10}, {30}).get(&baseValue, sizeof(baseValue), true);
    const auto attr2 = Const::ContentSetup(baseType).subview({0}, {30}).get(&baseValue, sizeof(baseValue), true);
    folding.enqueueRequest(attr1);
    folding.waitIdle();  // with two workers the equivalence request could otherwise overtake the fold of attr1
    folding.enqueueRequest(attr1, attr2);
    folding.waitIdle();
    EXPECT(folding.hasContent(attr2));
    EXPECT(!folding.hasContent(attr1));
    const vf_folder_stats st = folding.getStatistics();
    EXPECT(st.added == 2 && st.failed == 0 && st.hits == 1);
}

static void copyToTooSmall(const Context& ctx) {  // utils/content.cpp:172-174
    const TensorType baseType({4}, VF_DT_F32);
    const auto vals = generateValues<float>(4);
    bool thrown = false;
    try {
        (void)Const::ContentSetup(baseType).get(vals.data(), bytesOf(vals)).fold(ctx, 8);
    } catch (const Exception& e) {
        thrown = e.status() == VF_ERR_BUFFER_TOO_SMALL;
    }
    EXPECT(thrown);
}

int main(int argc, char** argv) {
    const bool hostOnly = argc > 1 && std::strcmp(argv[1], "--host") == 0;
    EXPECT(vf_abi_version() == VF_ABI_VERSION);
    positionRequirement();
    inferTypes();
    remainingTransformationTypes();
    optimizedLists();
    if (!hostOnly) {
        try {
            const Context ctx(0);
            quantize(ctx);
            dequantize(ctx);
            reorder(ctx);
            padWithZeroSplat(ctx);
            bitPack(ctx);
            getSparsityMap(ctx);
            sparsifyQuantized(ctx);
            dequantizeQuantize(ctx);
            relocateWeightsTable(ctx);
            copyToTooSmall(ctx);
            constantFoldingPass(ctx);
            foldingInBackground();
        } catch (const Exception& e) {
            std::printf("unexpected vfold::Exception %d: %s\n", e.status(), e.what());
            ++g_failed;
        }
    }
    std::printf("%s: %d failed check(s)\n", hostOnly ? "host" : "all", g_failed);
    return g_failed == 0 ? 0 : 1;
}
