// Per-op backends: dtype dispatch, ONNX shape inference, output allocation and the kernel call.
// One function per reference backend file (runtime/src/providers/cuda/backend/<op>.rs, cited at each).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>

#include "runtime.h"

namespace rmlk {
namespace rt {

namespace {

using Shape = std::vector<int64_t>;

bool is_int_dtype(int dt) {
    switch (dt) {
        case RMLK_I8: case RMLK_U8: case RMLK_I16: case RMLK_U16: case RMLK_I32: case RMLK_U32: case RMLK_I64: case RMLK_U64: case RMLK_BOOL:
            return true;
        default:
            return false;
    }
}
bool is_float_dtype(int dt) { return dt == RMLK_F16 || dt == RMLK_F32 || dt == RMLK_F64; }

bool in_set(int dt, std::initializer_list<int> s) { return std::find(s.begin(), s.end(), dt) != s.end(); }

int64_t prod(const Shape& s, size_t b = 0, size_t e = static_cast<size_t>(-1)) {
    if (e > s.size()) e = s.size();
    int64_t n = 1;
    for (size_t i = b; i < e; i++) n *= s[i];
    return n;
}

// Scalars are presented to kernels as shape [1] (reference runtime/src/providers/cuda/utils.rs:5-18).
Shape kshape(const Tensor& t) { return t.is_scalar() ? Shape{1} : t.shape; }

Shape dense_strides(const Shape& s) {
    Shape st(s.size(), 1);
    for (int i = static_cast<int>(s.size()) - 2; i >= 0; i--) st[i] = st[i + 1] * s[i + 1];
    return st;
}

// runtime/src/utils/mod.rs:114-143
bool broadcast_shape(const Shape& a, const Shape& b, Shape& out) {
    const size_t n = std::max(a.size(), b.size());
    out.assign(n, 1);
    for (size_t i = 0; i < n; i++) {
        const int64_t ad = i >= n - a.size() ? a[i - (n - a.size())] : 1;
        const int64_t bd = i >= n - b.size() ? b[i - (n - b.size())] : 1;
        if (ad != bd && ad != 1 && bd != 1) return false;
        out[i] = std::max(ad, bd);
        if (ad == 0 || bd == 0) out[i] = 0;
    }
    return true;
}

// runtime/src/utils/mod.rs:93-111: stride 0 wherever the operand is broadcast
Shape broadcast_strides(const Shape& shape, const Shape& out) {
    const Shape st = dense_strides(shape);
    Shape r(out.size(), 0);
    for (size_t i = 0; i < out.size(); i++) {
        if (i + shape.size() < out.size()) continue;
        const size_t j = i - (out.size() - shape.size());
        if (shape[j] == out[i] && shape[j] != 1) r[i] = st[j];
    }
    return r;
}

std::string shape_str(const Shape& s) {
    std::string r = "[";
    for (size_t i = 0; i < s.size(); i++) r += (i ? ", " : "") + std::to_string(s[i]);
    return r + "]";
}

// runtime/src/utils/mod.rs:159-182
int64_t normalize_index(int64_t index, int64_t size) {
    const int64_t n = index < 0 ? size + index : index;
    if (n < 0 || n > size) raise(RMLK_ERR_INVALID_ARG, "axis out of bound " + std::to_string(index));
    return n;
}

struct Ctx {
    Instance& I;
    const NodeDef& n;
    // Input i as it is: possibly a deferred view (Tensor::lazy).
    Tensor* raw(size_t i) const {
        if (i >= n.inputs.size() || n.inputs[i] < 0) return nullptr;
        Tensor& t = I.values[n.inputs[i]];
        if (!t.present) raise(RMLK_ERR_INVALID_ARG, "input value `" + I.g.values[n.inputs[i]].name + "` has no data");
        if (t.parts > 1) I.settle_parts(n.inputs[i]);
        return &t;
    }
    // Input i as a dense tensor; a deferred view is copied out first.
    Tensor* in(size_t i) const {
        Tensor* t = raw(i);
        if (t && t->lazy) I.materialize(*t);
        return t;
    }
    // May output i stay a view of another buffer?  Not if it leaves the graph or is carried to the next run.
    bool may_defer(size_t i) const {
        const int vid = n.outputs[i];
        return !I.g.values[vid].is_output && I.binding_of_out[vid] < 0;
    }
    Tensor& req(size_t i) const {
        Tensor* t = in(i);
        if (!t) raise(RMLK_ERR_INVALID_ARG, "missing input " + std::to_string(i));
        return *t;
    }
    Tensor& out(size_t i) const {
        if (i >= n.outputs.size()) raise(RMLK_ERR_INVALID_ARG, "missing output " + std::to_string(i));
        return I.values[n.outputs[i]];
    }
    const Attr* attr(const char* name) const {
        auto it = n.attrs.find(name);
        return it == n.attrs.end() ? nullptr : &it->second;
    }
    int64_t attr_int(const char* name, int64_t dflt) const {
        const Attr* a = attr(name);
        return (a && a->kind == Attr::INT) ? a->i : dflt;
    }
    // Allocate output i with the given dtype/shape (init_payload in the reference).
    Tensor& make(size_t i, int dtype, const Shape& shape) const {
        Tensor& o = out(i);
        o.dtype = dtype;
        o.shape = shape;
        o.mirror_valid = false;
        o.mi.clear();
        o.mf.clear();
        o.lazy = false;
        o.parts = 0;
        I.alloc_output(n.outputs[i], o);
        o.present = true;
        return o;
    }
    // Zero-copy view of `src` with a new shape (Reshape / Unsqueeze / Flatten).
    Tensor& view(size_t i, const Tensor& src, const Shape& shape) const {
        Tensor& o = out(i);
        const int vid = n.outputs[i];
        const bool bound = I.binding_of_out[vid] >= 0;
        o.dtype = src.dtype;
        o.shape = shape;
        o.mirror_valid = src.mirror_valid;
        o.mi = src.mi;
        o.mf = src.mf;
        o.parts = 0;
        if (bound) {  // a carried output must own its storage
            I.alloc_output(vid, o);
            if (o.nbytes()) check_cuda(cudaMemcpyAsync(o.data, src.data, o.nbytes(), cudaMemcpyDeviceToDevice, I.stream), "view copy");
            I.launches++;
        } else {
            o.data = src.data;
            o.storage = src.storage;
            if (o.storage) o.storage->refs++;
            // regrouping the dims of a deferred view leaves its element order, hence pshape / pstride, alone
            o.lazy = src.lazy;
            o.pshape = src.pshape;
            o.pstride = src.pstride;
        }
        o.present = true;
        return o;
    }
    // Output i becomes a deferred view of base's buffer: logical `shape`, elements enumerated by pshape / pstride.
    Tensor& defer(size_t i, const Tensor& base, const Shape& shape, const Shape& pshape, const Shape& pstride) const {
        Tensor& o = out(i);
        o.dtype = base.dtype;
        o.shape = shape;
        o.mirror_valid = false;
        o.mi.clear();
        o.mf.clear();
        o.parts = 0;
        o.data = base.data;
        o.storage = base.storage;
        if (o.storage) o.storage->refs++;
        // a permutation that only moves dims of size 1 (a [B, heads, 1, D] -> [B, 1, heads, D] transpose of one
        // decoded token) enumerates the buffer in its own order: that is an ordinary dense tensor, nothing deferred
        bool dense = true;
        int64_t expect = 1;
        for (size_t d = pshape.size(); d-- > 0 && dense;) {
            if (pshape[d] == 1) continue;
            dense = pstride[d] == expect;
            expect *= pshape[d];
        }
        o.lazy = !dense;
        if (dense) {
            o.pshape.clear();
            o.pstride.clear();
        } else {
            o.pshape = pshape;
            o.pstride = pstride;
        }
        o.present = true;
        return o;
    }
    rmlk_stream_t stream() const { return reinterpret_cast<rmlk_stream_t>(I.stream); }
    void launched(int k = 1) const { I.launches += k; }
};

// ---- host mirrors ---------------------------------------------------------------------------
void set_mirror_i(Tensor& t, const std::vector<int64_t>& v) {
    t.mi = v;
    t.mf.clear();
    t.mirror_valid = true;
}
void set_mirror_f(Tensor& t, const std::vector<double>& v) {
    t.mf = v;
    t.mi.clear();
    t.mirror_valid = true;
}
bool small_mirrored(const Tensor& t) { return t.mirror_valid && t.numel() <= HOST_MIRROR_MAX; }

double round_to(int dt, double v) {
    if (dt == RMLK_F32) return static_cast<double>(static_cast<float>(v));
    return v;  // f64 (f16 mirrors are not kept)
}

// Broadcasted element index helper for mirror arithmetic (all tensors are tiny).
int64_t bindex(const Shape& shape, const Shape& out, int64_t lin) {
    const Shape ost = dense_strides(out);
    const Shape st = broadcast_strides(shape, out);
    int64_t off = 0;
    for (size_t d = 0; d < out.size(); d++) {
        const int64_t c = (lin / ost[d]) % out[d];
        off += c * st[d];
    }
    return off;
}

// ---- deferred views -------------------------------------------------------------------------
// Physical dims of a tensor: pshape / pstride of a deferred view, else its shape with dense strides.
void phys_of(const Tensor& t, Shape& ps, Shape& pst) {
    if (t.lazy) {
        ps = t.pshape;
        pst = t.pstride;
    } else {
        ps = t.shape;
        pst = dense_strides(t.shape);
    }
}

// One run [begin, end) of consecutive physical dims per logical dim, products equal.  False when the edge
// of a logical dim falls inside a physical dim (the view was regrouped in a way the caller cannot follow).
bool group_dims(const Shape& logical, const Shape& ps, std::vector<std::pair<int, int>>& groups) {
    groups.clear();
    int p = 0;
    const int np = static_cast<int>(ps.size());
    for (size_t d = 0; d < logical.size(); d++) {
        const int begin = p;
        int64_t run = 1;
        if (logical[d] <= 0) return false;
        while (run < logical[d]) {
            if (p >= np) return false;
            run *= ps[p++];
        }
        if (run != logical[d]) return false;
        groups.push_back({begin, p});
    }
    for (; p < np; p++)
        if (ps[p] != 1) return false;
    return true;
}

void push_dim(Shape& ps, Shape& pst, int64_t size, int64_t stride) {
    if (size == 1) return;
    ps.push_back(size);
    pst.push_back(stride);
}

// Splits physical dims where an edge of a logical dim falls inside one and divides it evenly (a dim of size
// a * b and stride s is the two dims (a, s * b), (b, s)), so that afterwards every logical dim is a run of whole
// physical dims.  False (ps / pst untouched) when some edge does not divide.
bool refine_dims(const Shape& logical, Shape& ps, Shape& pst) {
    Shape nps, npst;
    size_t p = 0;
    int64_t rem = 1, rstride = 0;
    auto next = [&]() {
        if (p >= ps.size()) return false;
        rem = ps[p];
        rstride = pst[p];
        p++;
        return true;
    };
    for (int64_t n : logical) {
        if (n <= 0) return false;
        int64_t need = n;
        while (need > 1) {
            if (rem == 1 && !next()) return false;
            if (rem == 1) continue;
            if (need >= rem) {
                if (need % rem) return false;
                push_dim(nps, npst, rem, rstride);
                need /= rem;
                rem = 1;
            } else {
                if (rem % need) return false;
                push_dim(nps, npst, need, rstride * (rem / need));
                rem /= need;
                need = 1;
            }
        }
    }
    if (rem != 1) return false;
    for (; p < ps.size(); p++)
        if (ps[p] != 1) return false;
    ps = nps;
    pst = npst;
    return true;
}

// Physical dims of `t`, refined to its logical shape, and the run of physical dims behind each logical dim.
bool dims_of(const Tensor& t, Shape& ps, Shape& pst, std::vector<std::pair<int, int>>& groups) {
    phys_of(t, ps, pst);
    if (t.lazy) refine_dims(t.shape, ps, pst);
    return group_dims(t.shape, ps, groups);
}

// A deferred right operand of MatMul that is a dense [k, n] (or, transposed, a dense [n, k]) matrix per
// batch entry, whose batch dims are `outer` entries `sb` elements apart followed by `fold` entries that
// all read the same matrix (stride 0: a broadcast such as grouped-query attention's repeated KV heads).
struct LazyB {
    bool transposed = false;
    int64_t outer = 1, fold = 1, sb = 0;
};
bool analyze_lazy_b(const Tensor& b, int64_t k, int64_t n, LazyB& r) {
    const size_t br = b.shape.size();
    if (br < 2) return false;
    std::vector<std::pair<int, int>> groups;
    Shape ps, pst;
    if (!dims_of(b, ps, pst, groups)) return false;
    auto single = [&](const std::pair<int, int>& g, int64_t& stride) {
        int cnt = 0;
        stride = 0;
        for (int p = g.first; p < g.second; p++)
            if (ps[p] != 1) {
                cnt++;
                stride = pst[p];
            }
        return cnt <= 1;
    };
    int64_t sk = 0, sn = 0;
    if (!single(groups[br - 2], sk) || !single(groups[br - 1], sn)) return false;
    const bool nn = (n == 1 || sn == 1) && (k == 1 || sk == n);
    const bool nt = (k == 1 || sk == 1) && (n == 1 || sn == k);
    if (!nn && !nt) return false;
    r.transposed = !nn;
    Shape bd, bs;
    for (size_t d = 0; d + 2 < br; d++)
        for (int p = groups[d].first; p < groups[d].second; p++) push_dim(bd, bs, ps[p], pst[p]);
    r.fold = 1;
    while (!bd.empty() && bs.back() == 0) {
        r.fold *= bd.back();
        bd.pop_back();
        bs.pop_back();
    }
    r.outer = 1;
    r.sb = 0;
    if (!bd.empty()) {
        r.sb = bs.back();
        for (size_t i = bd.size(); i-- > 0;) {
            if (i + 1 < bd.size() && bs[i] != bs[i + 1] * bd[i + 1]) return false;
            r.outer *= bd[i];
        }
        if (r.sb <= 0) return false;
    }
    return true;
}

// ---------------------------------------------------------------------------------------------
// broadcast elementwise family
// ---------------------------------------------------------------------------------------------
// backend/binary.rs:18-162 with backend/{add,sub,mul,div,equal,greater}.rs
void op_binary(const Ctx& c, int bop) {
    Tensor& a = c.req(0);
    Tensor& b = c.req(1);
    if (!in_set(a.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64})) unsupported_dtype(a.dtype, "binary op");
    if (a.dtype != b.dtype) raise(RMLK_ERR_INVALID_ARG, "binary op: operand data types differ (" + dtype_name(a.dtype) + " vs " + dtype_name(b.dtype) + ")");
    Shape oshape;
    if (!broadcast_shape(a.shape, b.shape, oshape))
        raise(RMLK_ERR_INVALID_ARG, "incompatible tensor shapes: " + shape_str(a.shape) + " " + shape_str(b.shape));
    const bool cmp = bop == RMLK_BIN_EQUAL || bop == RMLK_BIN_GREATER;
    Tensor& o = c.make(0, cmp ? RMLK_BOOL : a.dtype, oshape);
    const Shape ks = (a.is_scalar() && b.is_scalar()) ? Shape{1} : oshape;
    const Shape as = broadcast_strides(kshape(a), ks), bs = broadcast_strides(kshape(b), ks);
    check_rc(rmlk_b200_binary(c.stream(), bop, a.dtype, static_cast<int>(ks.size()), ks.data(), as.data(), bs.data(), a.data, b.data, o.data));
    c.launched();
    if (small_mirrored(a) && small_mirrored(b) && o.numel() <= HOST_MIRROR_MAX && a.dtype != RMLK_F16) {
        const int64_t n = o.numel();
        const bool isf = is_float_dtype(a.dtype);
        std::vector<int64_t> ri(isf && !cmp ? 0 : n);
        std::vector<double> rf(isf && !cmp ? n : 0);
        for (int64_t i = 0; i < n; i++) {
            const int64_t ia = bindex(a.shape, oshape, i), ib = bindex(b.shape, oshape, i);
            if (isf) {
                const double x = a.mf[ia], y = b.mf[ib];
                switch (bop) {
                    case RMLK_BIN_ADD: rf[i] = round_to(a.dtype, x + y); break;
                    case RMLK_BIN_SUB: rf[i] = round_to(a.dtype, x - y); break;
                    case RMLK_BIN_MUL: rf[i] = round_to(a.dtype, x * y); break;
                    case RMLK_BIN_DIV: rf[i] = round_to(a.dtype, x / y); break;
                    case RMLK_BIN_EQUAL: ri[i] = x == y; break;
                    default: ri[i] = x > y; break;
                }
            } else {
                const int64_t x = a.mi[ia], y = b.mi[ib];
                auto wrap = [&](int64_t v) { return a.dtype == RMLK_I32 ? static_cast<int64_t>(static_cast<int32_t>(v)) : v; };
                switch (bop) {
                    case RMLK_BIN_ADD: ri[i] = wrap(static_cast<int64_t>(static_cast<uint64_t>(x) + static_cast<uint64_t>(y))); break;
                    case RMLK_BIN_SUB: ri[i] = wrap(static_cast<int64_t>(static_cast<uint64_t>(x) - static_cast<uint64_t>(y))); break;
                    case RMLK_BIN_MUL: ri[i] = wrap(static_cast<int64_t>(static_cast<uint64_t>(x) * static_cast<uint64_t>(y))); break;
                    case RMLK_BIN_DIV: ri[i] = (y == 0 || (x == std::numeric_limits<int64_t>::min() && y == -1)) ? 0 : wrap(x / y); break;
                    case RMLK_BIN_EQUAL: ri[i] = x == y; break;
                    default: ri[i] = x > y; break;
                }
            }
        }
        if (isf && !cmp) set_mirror_f(o, rf); else set_mirror_i(o, ri);
    }
}

// backend/pow.rs:95-132
void op_pow(const Ctx& c) {
    Tensor& a = c.req(0);
    Tensor& b = c.req(1);
    if (!in_set(a.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64})) unsupported_dtype(a.dtype, "pow base");
    if (!in_set(b.dtype, {RMLK_U8, RMLK_U16, RMLK_U32, RMLK_U64, RMLK_I8, RMLK_I16, RMLK_I32, RMLK_I64, RMLK_F16, RMLK_F32, RMLK_F64}))
        unsupported_dtype(b.dtype, "pow exponent");
    Shape oshape;
    if (!broadcast_shape(a.shape, b.shape, oshape))
        raise(RMLK_ERR_INVALID_ARG, "incompatible tensor shapes: " + shape_str(a.shape) + " " + shape_str(b.shape));
    Tensor& o = c.make(0, a.dtype, oshape);
    const Shape ks = (a.is_scalar() && b.is_scalar()) ? Shape{1} : oshape;
    const Shape as = broadcast_strides(kshape(a), ks), bs = broadcast_strides(kshape(b), ks);
    check_rc(rmlk_b200_pow(c.stream(), a.dtype, b.dtype, static_cast<int>(ks.size()), ks.data(), as.data(), bs.data(), a.data, b.data, o.data));
    c.launched();
}

// backend/unary.rs:12-50 (+ sqrt/neg/sin/cos.rs); backend/activation.rs:30-155 (sigmoid.rs, relu.rs)
void op_unary(const Ctx& c, int uop) {
    Tensor& x = c.req(0);
    const bool ints_ok = uop == RMLK_UN_NEG || uop == RMLK_UN_RELU;
    if (!(is_float_dtype(x.dtype) || (ints_ok && in_set(x.dtype, {RMLK_I32, RMLK_I64})))) unsupported_dtype(x.dtype, "unary op");
    Tensor& o = c.make(0, x.dtype, x.shape);
    check_rc(rmlk_b200_unary(c.stream(), uop, x.dtype, static_cast<size_t>(x.numel()), x.data, o.data));
    c.launched();
    if (uop == RMLK_UN_NEG && small_mirrored(x) && x.dtype != RMLK_F16) {
        if (is_float_dtype(x.dtype)) {
            std::vector<double> r(x.mf);
            for (double& v : r) v = -v;
            set_mirror_f(o, r);
        } else {
            std::vector<int64_t> r(x.mi);
            for (int64_t& v : r) v = -v;
            set_mirror_i(o, r);
        }
    }
}

int onnx_to_dtype(int64_t code) {
    switch (code) {
        case 1: return RMLK_F32; case 2: return RMLK_U8; case 3: return RMLK_I8; case 4: return RMLK_U16; case 5: return RMLK_I16;
        case 6: return RMLK_I32; case 7: return RMLK_I64; case 8: return RMLK_STRING; case 9: return RMLK_BOOL; case 10: return RMLK_F16;
        case 11: return RMLK_F64; case 12: return RMLK_U32; case 13: return RMLK_U64;
        default: raise(RMLK_ERR_INVALID_ARG, "cast: unknown data type code " + std::to_string(code));
    }
}

int64_t wrap_int(int dt, int64_t v) {
    switch (dt) {
        case RMLK_I8: return static_cast<int8_t>(v); case RMLK_U8: return static_cast<uint8_t>(v);
        case RMLK_I16: return static_cast<int16_t>(v); case RMLK_U16: return static_cast<uint16_t>(v);
        case RMLK_I32: return static_cast<int32_t>(v); case RMLK_U32: return static_cast<uint32_t>(v);
        case RMLK_BOOL: return v != 0;
        default: return v;
    }
}

// backend/cast.rs:29-179
void op_cast(const Ctx& c) {
    Tensor& x = c.req(0);
    const Attr* to = c.attr("to");
    if (!to || to->kind != Attr::INT) raise(RMLK_ERR_INVALID_ARG, "missing `to` cast attribute");
    const int dst = onnx_to_dtype(to->i);
    // The op accepts the pairs the reference's backend dispatches (backend/cast.rs:30-67) and rejects the
    // rest with the same "unsupported" error, although the kernel launcher takes every pair.
    {
        const int s = x.dtype;
        const bool sf = is_float_dtype(s), df = is_float_dtype(dst);
        const bool s4 = in_set(s, {RMLK_I32, RMLK_U32, RMLK_I64, RMLK_U64}), d4 = in_set(dst, {RMLK_I32, RMLK_U32, RMLK_I64, RMLK_U64});
        bool ok = (sf && (df || d4) && s != dst) || (s4 && df);
        ok = ok || (s == RMLK_I32 && dst == RMLK_I64) || (s == RMLK_I64 && dst == RMLK_I32) || (s == RMLK_U32 && dst == RMLK_U64) ||
             (s == RMLK_U64 && dst == RMLK_U32) || (s == RMLK_BOOL && dst == RMLK_F32);
        if (!ok) raise(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported cast: " + dtype_name(s) + " -> " + dtype_name(dst));
    }
    Tensor& o = c.make(0, dst, x.shape);
    check_rc(rmlk_b200_cast(c.stream(), x.dtype, dst, static_cast<size_t>(x.numel()), x.data, o.data));
    c.launched();
    if (small_mirrored(x) && x.dtype != RMLK_F16 && dst != RMLK_F16) {
        const int64_t n = x.numel();
        if (is_float_dtype(dst)) {
            std::vector<double> r(n);
            for (int64_t i = 0; i < n; i++) r[i] = round_to(dst, is_float_dtype(x.dtype) ? x.mf[i] : static_cast<double>(x.mi[i]));
            set_mirror_f(o, r);
        } else {
            std::vector<int64_t> r(n);
            bool ok = true;
            for (int64_t i = 0; i < n; i++) {
                if (is_float_dtype(x.dtype)) {
                    const double v = x.mf[i];
                    if (!(std::fabs(v) < 9.0e18)) { ok = false; break; }  // saturating / NaN cases: leave to the device
                    r[i] = dst == RMLK_BOOL ? (v != 0.0) : wrap_int(dst, static_cast<int64_t>(v));
                } else {
                    r[i] = wrap_int(dst, x.mi[i]);
                }
            }
            if (ok) set_mirror_i(o, r);
        }
    }
}

// backend/whereop.rs:43-264
void op_where(const Ctx& c) {
    Tensor& cond = c.req(0);
    Tensor& x = c.req(1);
    Tensor& y = c.req(2);
    if (!in_set(x.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64})) unsupported_dtype(x.dtype, "where");
    if (cond.dtype != RMLK_BOOL) raise(RMLK_ERR_INVALID_ARG, "where: condition must be a bool tensor");
    if (x.dtype != y.dtype) raise(RMLK_ERR_INVALID_ARG, "where: x and y data types differ");
    Shape inter, oshape;
    if (!broadcast_shape(x.shape, y.shape, inter) || !broadcast_shape(inter, cond.shape, oshape))
        raise(RMLK_ERR_INVALID_ARG, "incompatible shapes for broadcast: " + shape_str(x.shape) + " " + shape_str(y.shape) + " " + shape_str(cond.shape));
    Tensor& o = c.make(0, x.dtype, oshape);
    const Shape ks = oshape.empty() ? Shape{1} : oshape;
    const Shape xs = broadcast_strides(kshape(x), ks), ys = broadcast_strides(kshape(y), ks), cs = broadcast_strides(kshape(cond), ks);
    check_rc(rmlk_b200_where(c.stream(), x.dtype, static_cast<int>(ks.size()), ks.data(), xs.data(), ys.data(), cs.data(), x.data, y.data, cond.data, o.data));
    c.launched();
    if (small_mirrored(x) && small_mirrored(y) && small_mirrored(cond) && o.numel() <= HOST_MIRROR_MAX && x.dtype != RMLK_F16) {
        const int64_t n = o.numel();
        const bool isf = is_float_dtype(x.dtype);
        std::vector<int64_t> ri(isf ? 0 : n);
        std::vector<double> rf(isf ? n : 0);
        for (int64_t i = 0; i < n; i++) {
            const bool z = cond.mi[bindex(cond.shape, oshape, i)] != 0;
            const int64_t ix = bindex(x.shape, oshape, i), iy = bindex(y.shape, oshape, i);
            if (isf) rf[i] = z ? x.mf[ix] : y.mf[iy]; else ri[i] = z ? x.mi[ix] : y.mi[iy];
        }
        if (isf) set_mirror_f(o, rf); else set_mirror_i(o, ri);
    }
}

// ---------------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------------
// backend/reduce_mean.rs:47-310
void op_reduce_mean(const Ctx& c) {
    Tensor& x = c.req(0);
    if (!in_set(x.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64})) unsupported_dtype(x.dtype, "reduce_mean");
    const int64_t rank = x.is_scalar() ? 1 : static_cast<int64_t>(x.shape.size());
    const bool noop = c.attr_int("noop_with_empty_axes", 0) > 0;
    const bool keepdims = c.attr_int("keepdims", 1) > 0;
    bool have_axes = false;
    std::vector<int64_t> axes;
    if (Tensor* at = c.in(1)) {
        if (at->numel() > 0) {
            for (int64_t v : c.I.host_i64(*at)) axes.push_back(normalize_index(v, rank));
            have_axes = true;
        } else if (at->is_scalar()) {
            raise(RMLK_ERR_INVALID_ARG, "ScalarAxisNotAllowed");
        }
    } else if (const Attr* a = c.attr("axes")) {
        if (a->kind == Attr::INTS && !a->ints.empty()) {
            for (int64_t v : a->ints) axes.push_back(normalize_index(v, rank));
            have_axes = true;
        }
    } else {
        for (int64_t i = 0; i < rank; i++) axes.push_back(i);
        have_axes = true;
    }
    if (!have_axes && noop) {  // copy the input (copy_input_to_output, reduce_mean.rs:229-244)
        Tensor& o = c.make(0, x.dtype, x.shape);
        if (o.nbytes()) check_cuda(cudaMemcpyAsync(o.data, x.data, o.nbytes(), cudaMemcpyDeviceToDevice, c.I.stream), "reduce_mean copy");
        c.launched();
        return;
    }
    if (!have_axes) for (int64_t i = 0; i < rank; i++) axes.push_back(i);
    std::vector<bool> reduced(rank, false);
    for (int64_t a : axes) {
        if (a >= rank) raise(RMLK_ERR_INVALID_ARG, "AxisOutOfBounds");
        if (reduced[a]) raise(RMLK_ERR_INVALID_ARG, "DuplicateAxis");
        reduced[a] = true;
    }
    Shape oshape;
    if (!x.is_scalar()) {
        if (!keepdims && static_cast<int64_t>(axes.size()) > rank) raise(RMLK_ERR_INVALID_ARG, "AxesLargerThanRank");
        for (int64_t d = 0; d < rank; d++) {
            if (reduced[d]) { if (keepdims) oshape.push_back(1); }
            else oshape.push_back(x.shape[d]);
        }
    }
    Tensor& o = c.make(0, x.dtype, oshape);
    const Shape ks = kshape(x);
    if (x.numel() == 0) return;
    check_rc(rmlk_b200_reduce_mean(c.stream(), x.dtype, static_cast<int>(ks.size()), ks.data(), static_cast<int>(axes.size()), axes.data(), x.data, o.data));
    c.launched();
}

// backend/softmax.rs:31-158
void op_softmax(const Ctx& c) {
    Tensor& x = c.req(0);
    if (x.dtype != RMLK_F32) unsupported_dtype(x.dtype, "softmax");
    const int64_t axis = c.attr_int("axis", -1);
    const int64_t rank = static_cast<int64_t>(x.shape.size());
    if (!(axis == -1 || (axis == 1 && rank == 4)))
        raise(RMLK_ERR_INVALID_ARG, "unsupported input values: unsupported inputs axis `" + std::to_string(axis) + "` and rank `" + std::to_string(rank) + "`");
    if (rank == 0) raise(RMLK_ERR_INVALID_ARG, "softmax: scalar input");
    Tensor& o = c.make(0, x.dtype, x.shape);
    if (axis == -1) {
        const int64_t cols = x.shape[rank - 1];
        check_rc(rmlk_b200_softmax(c.stream(), x.dtype, cols ? x.numel() / cols : 0, cols, x.data, o.data));
    } else {
        check_rc(rmlk_b200_softmax_strided(c.stream(), x.dtype, x.shape[0], x.shape[1], x.shape[2] * x.shape[3], x.data, o.data));
    }
    c.launched();
}

// ---------------------------------------------------------------------------------------------
// MatMul — backend/matmul.rs:223-356
// ---------------------------------------------------------------------------------------------
// ONNX Gemm: Y = alpha * op(A) * op(B) + beta * C for rank-2 A and B (backend/gemm.rs:149-216).  C broadcasts to [M, N] by the ONNX
// rule (a vector of N entries is a row, a vector of M entries a column - the reference's two 1-D cases, backend/gemm.rs:225-227).
void op_gemm(const Ctx& c) {
    Tensor& a = c.req(0);
    Tensor& b = c.req(1);
    Tensor* bias = c.n.inputs.size() > 2 ? c.in(2) : nullptr;
    if (!in_set(a.dtype, {RMLK_F32, RMLK_F16})) unsupported_dtype(a.dtype, "gemm");
    if (b.dtype != a.dtype || (bias && bias->dtype != a.dtype)) raise(RMLK_ERR_INVALID_ARG, "gemm: operand data types differ");
    if (a.shape.size() != 2 || b.shape.size() != 2) raise(RMLK_ERR_INVALID_ARG, "expected inputs with rank 2");
    const bool ta = c.attr_int("transA", 0) != 0, tb = c.attr_int("transB", 0) != 0;
    const Attr* aa = c.attr("alpha");
    const Attr* ab = c.attr("beta");
    const float alpha = (aa && aa->kind == Attr::FLOAT) ? aa->f : 1.f, beta = (ab && ab->kind == Attr::FLOAT) ? ab->f : 1.f;
    const int64_t m = ta ? a.shape[1] : a.shape[0], k = ta ? a.shape[0] : a.shape[1];
    const int64_t kb = tb ? b.shape[1] : b.shape[0], n = tb ? b.shape[0] : b.shape[1];
    if (k != kb) raise(RMLK_ERR_INVALID_ARG, "IncompatibleDimForMul");
    int64_t cs_row = 0, cs_col = 0;
    if (bias) {
        const Shape& s = bias->shape;
        if (s.empty() || (s.size() == 1 && s[0] == 1)) { cs_row = cs_col = 0; }
        else if (s.size() == 1 && s[0] == n) { cs_row = 0; cs_col = 1; }
        else if (s.size() == 1 && s[0] == m) { cs_row = 1; cs_col = 0; }
        else if (s.size() == 2 && (s[0] == m || s[0] == 1) && (s[1] == n || s[1] == 1)) { cs_row = s[0] == 1 ? 0 : s[1]; cs_col = s[1] == 1 ? 0 : 1; }
        else raise(RMLK_ERR_INVALID_ARG, "invalid tensor shape");
    }
    Tensor& y = c.make(0, a.dtype, Shape({m, n}));
    if (y.numel() == 0) return;
    const size_t es = dtype_size_of(a.dtype);
    const void* ap = a.data;
    Storage* at = nullptr;
    if (ta) {  // [k, m] -> [m, k]
        at = c.I.arena->alloc(static_cast<size_t>(m) * k * es);
        const int64_t perm[2] = {1, 0};
        check_rc(rmlk_b200_transpose(c.stream(), static_cast<int>(es), 2, a.shape.data(), perm, a.data, at->ptr));
        c.launched();
        ap = at->ptr;
    }
    Storage* bt = nullptr;
    if (tb && a.dtype == RMLK_F32) {
        check_rc(rmlk_b200_matmul_nt(c.stream(), a.dtype, 1, m, n, k, ap, 0, b.data, 0, y.data, 0));  // B stored [n, k]: read as it lies
        c.launched();
    } else {
        const void* bp = b.data;
        if (tb) {
            bt = c.I.arena->alloc(static_cast<size_t>(n) * k * es);
            const int64_t perm[2] = {1, 0};
            check_rc(rmlk_b200_transpose(c.stream(), static_cast<int>(es), 2, b.shape.data(), perm, b.data, bt->ptr));
            c.launched();
            bp = bt->ptr;
        }
        const size_t need = rmlk_b200_matmul_workspace_bytes(a.dtype, 1, m, n, k);
        void* ws = need ? c.I.matmul_ws.ensure(need) : nullptr;
        const int flags = (!tb && c.I.g.values[c.n.inputs[1]].is_const) ? RMLK_MATMUL_B_STATIC : 0;
        check_rc(rmlk_b200_matmul_flags(c.stream(), a.dtype, 1, m, n, k, ap, 0, bp, 0, y.data, 0, ws, need, static_cast<int*>(c.I.status_word.ptr), flags));
        c.I.status_dirty = true;
        c.launched();
    }
    if (at) c.I.arena->release(at);
    if (bt) c.I.arena->release(bt);
    if (alpha != 1.f || bias) {
        check_rc(rmlk_b200_scale_add_bias(c.stream(), a.dtype, m, n, y.data, alpha, bias ? bias->data : nullptr, cs_row, cs_col, beta));
        c.launched();
    }
}

void op_matmul(const Ctx& c) {
    Tensor& a = c.req(0);
    Tensor* braw = c.raw(1);
    if (!braw) raise(RMLK_ERR_INVALID_ARG, "missing input 1");
    Tensor& b = *braw;  // may be a deferred view; made dense below unless the kernels can read it as it is
    if (!in_set(a.dtype, {RMLK_F32, RMLK_F16})) unsupported_dtype(a.dtype, "matmul");
    if (b.dtype != a.dtype) raise(RMLK_ERR_INVALID_ARG, "matmul: operand data types differ");
    const size_t ar = a.shape.size(), br = b.shape.size();
    if (ar == 0 || br == 0) raise(RMLK_ERR_INVALID_ARG, "ZeroRank");
    const int64_t m = ar == 1 ? 1 : a.shape[ar - 2], ka = a.shape[ar - 1];
    const int64_t kb = br == 1 ? b.shape[0] : b.shape[br - 2], n = br == 1 ? 1 : b.shape[br - 1];
    const int64_t ba = ar > 2 ? prod(a.shape, 0, ar - 2) : 1, bb = br > 2 ? prod(b.shape, 0, br - 2) : 1;
    if (ka != kb) raise(RMLK_ERR_INVALID_ARG, "IncompatibleDimForMul");
    if (ba != bb && ba != 1 && bb != 1) raise(RMLK_ERR_INVALID_ARG, "IncompatibleDimForBroadcast");
    const int64_t batch = std::max(ba, bb);
    // Output shape: NumPy matmul.  (The reference collapses the leading batch dims of rank >= 3 results
    // into one, matmul.rs:321-333; the buffer contents are identical.)
    Shape lead;
    if (ar > 2 && (ba >= bb || br <= 2)) lead.assign(a.shape.begin(), a.shape.end() - 2);
    else if (br > 2) lead.assign(b.shape.begin(), b.shape.end() - 2);
    Shape oshape = lead;
    if (ar > 1) oshape.push_back(m);
    if (br > 1) oshape.push_back(n);
    Tensor& o = c.make(0, a.dtype, oshape);
    if (o.numel() == 0) return;
    if (b.lazy) {
        // Right operand still a view (Expand / Reshape / Transpose chain).  If it is a dense matrix per batch
        // entry, possibly transposed, possibly repeated over trailing batch dims, the kernels read the
        // base buffer directly: the repeats become extra rows of A (they share one B), the transposition
        // selects the A x B^T kernel.  Otherwise it is copied out once and the dense path below runs.
        LazyB lb;
        bool usable = a.dtype == RMLK_F32 && ar >= 2 && br >= 2 && (ba == bb || bb == 1) && ka > 0 && analyze_lazy_b(b, kb, n, lb) && lb.outer * lb.fold == bb;
        const int64_t em = usable ? (bb == 1 ? ba : lb.fold) * m : 0;  // one shared B: every batch entry of A is extra rows
        usable = usable && (!lb.transposed || (em <= 8 && ka <= 128 && ka % 4 == 0));
        if (usable) {
            if (lb.transposed) {
                check_rc(rmlk_b200_matmul_nt(c.stream(), a.dtype, lb.outer, em, n, ka, a.data, em * ka, b.data, lb.sb, o.data, em * n));
                c.launched();
            } else {
                const size_t need = rmlk_b200_matmul_workspace_bytes(a.dtype, lb.outer, em, n, ka);
                void* ws = need ? c.I.matmul_ws.ensure(need) : nullptr;
                check_rc(rmlk_b200_matmul_ex(c.stream(), a.dtype, lb.outer, em, n, ka, a.data, em * ka, b.data, lb.sb, o.data, em * n, ws, need,
                                             static_cast<int*>(c.I.status_word.ptr)));
                c.I.status_dirty = true;
                c.launched(need ? 2 : 1);
            }
            return;
        }
        c.I.materialize(b);
    }
    // A weight shared by every batch entry (rank <= 2 right operand) folds the batch into M: one
    // pass over B instead of the reference's per-batch copies (matmul.rs:48-86).
    int64_t eb = batch, em = m, sa = ba > 1 ? m * ka : 0, sb = bb > 1 ? kb * n : 0, sc = m * n;
    if (bb == 1 && ba > 1) {
        em = ba * m;
        eb = 1;
        sa = sb = 0;
        sc = em * n;
    }
    const size_t need = rmlk_b200_matmul_workspace_bytes(a.dtype, eb, em, n, ka);
    const int ovid = c.n.outputs[0];
    // initializers were uploaded before the first run: nothing in flight writes them
    const int flags = c.I.g.values[c.n.inputs[1]].is_const ? RMLK_MATMUL_B_STATIC : 0;
    if (need && a.dtype == RMLK_F32 && eb == 1 && c.I.parts_owner < 0 && ovid < static_cast<int>(c.I.parts_ok_value.size()) && c.I.parts_ok_value[ovid]) {
        // The only reader is a residual Add + RMSNorm chain whose kernel adds split-K slabs itself: leave them unreduced.
        void* slabs = c.I.parts_ws.ensure(need);
        int parts = 1;
        check_rc(rmlk_b200_matmul_parts(c.stream(), a.dtype, em, n, ka, a.data, b.data, o.data, slabs, need, static_cast<int*>(c.I.status_word.ptr),
                                        flags, &parts));
        c.I.status_dirty = true;
        c.launched();
        if (parts > 1) {
            c.I.release_value(ovid);  // the dense buffer is not needed unless the chain falls back (settle_parts)
            o.data = slabs;
            o.parts = parts;
            c.I.parts_owner = ovid;
        }
        return;
    }
    const int hout = c.I.host_output_of(ovid);
    if (hout >= 0 && !need && a.dtype == RMLK_F32 && eb == 1 && n % 128 == 0 && c.I.host_outputs[hout].nbytes == o.nbytes()) {
        // An output the host is waiting for (logits): the product is issued in blocks of columns - one wave of tiles,
        // then two waves each - and every block goes to the host on the copy stream while the next is computed.
        int sm_attr = 148;
        cudaDeviceGetAttribute(&sm_attr, cudaDevAttrMultiProcessorCount, c.I.device);
        const int64_t sms = sm_attr > 0 ? sm_attr : 148, tiles = n / 128;
        std::vector<int64_t> blocks;
        for (int64_t left = tiles, first = 1; left > 0; first = 0) {
            int64_t take = std::min<int64_t>(left, first ? sms : 2 * sms);
            if (left - take < sms) take = left;  // a short tail joins the last block
            blocks.push_back(take);
            left -= take;
        }
        bool ok = blocks.size() > 1;
        for (int64_t bt : blocks) ok = ok && rmlk_b200_matmul_window_supported(em, bt * 128, ka, n);
        if (ok) {
            HostOutput& h = c.I.host_outputs[hout];
            while (c.I.copy_events.size() < blocks.size()) {
                cudaEvent_t e = nullptr;
                check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
                c.I.copy_events.push_back(e);
            }
            int64_t n0 = 0;
            for (size_t i = 0; i < blocks.size(); i++) {
                const int64_t nc = blocks[i] * 128;
                check_rc(rmlk_b200_matmul_window(c.stream(), a.dtype, em, nc, ka, a.data, static_cast<const float*>(b.data) + n0,
                                                 static_cast<float*>(o.data) + n0, n, static_cast<int*>(c.I.status_word.ptr), flags));
                check_cuda(cudaEventRecord(c.I.copy_events[i], c.I.stream), "cudaEventRecord");
                check_cuda(cudaStreamWaitEvent(c.I.copy_stream, c.I.copy_events[i], 0), "cudaStreamWaitEvent");
                check_cuda(cudaMemcpy2DAsync(static_cast<char*>(h.dst) + n0 * 4, static_cast<size_t>(n) * 4, static_cast<const float*>(o.data) + n0,
                                             static_cast<size_t>(n) * 4, static_cast<size_t>(nc) * 4, static_cast<size_t>(em), cudaMemcpyDeviceToHost,
                                             c.I.copy_stream), "host output D2H");
                n0 += nc;
            }
            h.delivered_run = c.I.run_counter;
            c.I.copies_pending = true;
            c.I.status_dirty = true;
            c.launched(static_cast<int>(blocks.size()));
            return;
        }
    }
    void* ws = need ? c.I.matmul_ws.ensure(need) : nullptr;
    check_rc(rmlk_b200_matmul_flags(c.stream(), a.dtype, eb, em, n, ka, a.data, sa, b.data, sb, o.data, sc, ws, need,
                                    static_cast<int*>(c.I.status_word.ptr), flags));
    c.I.status_dirty = true;
    c.launched(need ? 2 : 1);
}

// ---------------------------------------------------------------------------------------------
// indexing / layout
// ---------------------------------------------------------------------------------------------
// backend/gather.rs:28-258
void op_gather(const Ctx& c) {
    Tensor& data = c.req(0);
    Tensor& idx = c.req(1);
    if (!in_set(data.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_U32, RMLK_I64, RMLK_U64})) unsupported_dtype(data.dtype, "gather");
    if (!in_set(idx.dtype, {RMLK_I32, RMLK_I64})) unsupported_dtype(idx.dtype, "gather indices");
    if (data.is_scalar()) raise(RMLK_ERR_INVALID_ARG, "scalar input data not allowed");
    const int64_t rank = static_cast<int64_t>(data.shape.size());
    const int64_t axis = normalize_index(c.attr_int("axis", 0), rank);
    if (axis >= rank) raise(RMLK_ERR_INVALID_ARG, "rank axis mismatch");
    Shape oshape(data.shape.begin(), data.shape.begin() + axis);
    oshape.insert(oshape.end(), idx.shape.begin(), idx.shape.end());
    oshape.insert(oshape.end(), data.shape.begin() + axis + 1, data.shape.end());
    const int64_t axis_dim = data.shape[axis];
    if (small_mirrored(idx)) {  // host-visible indices are validated up front, as the reference does for all of them
        for (int64_t v : idx.mi)
            if (v < -axis_dim || v >= axis_dim) raise(RMLK_ERR_INVALID_ARG, "axis out of bound " + std::to_string(v));
    }
    Tensor& o = c.make(0, data.dtype, oshape);
    const int64_t outer = prod(data.shape, 0, axis), inner = prod(data.shape, axis + 1);
    check_rc(rmlk_b200_gather(c.stream(), static_cast<int>(dtype_size_of(data.dtype)), idx.dtype, outer, axis_dim, inner, idx.numel(), data.data,
                              idx.data, o.data, static_cast<int*>(c.I.status_word.ptr)));
    c.launched();
    if (small_mirrored(data) && small_mirrored(idx) && o.numel() <= HOST_MIRROR_MAX && data.dtype != RMLK_F16) {
        const int64_t n_idx = idx.numel();
        const bool isf = is_float_dtype(data.dtype);
        std::vector<int64_t> ri;
        std::vector<double> rf;
        for (int64_t ou = 0; ou < outer; ou++)
            for (int64_t j = 0; j < n_idx; j++) {
                int64_t ix = idx.mi[j];
                if (ix < 0) ix += axis_dim;
                for (int64_t e = 0; e < inner; e++) {
                    const int64_t src = (ou * axis_dim + ix) * inner + e;
                    if (isf) rf.push_back(data.mf[src]); else ri.push_back(data.mi[src]);
                }
            }
        if (isf) set_mirror_f(o, rf); else set_mirror_i(o, ri);
    }
}

// backend/scatter_nd.rs:30-210
void op_scatter_nd(const Ctx& c) {
    Tensor& data = c.req(0);
    Tensor& idx = c.req(1);
    Tensor& upd = c.req(2);
    if (!in_set(data.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64})) unsupported_dtype(data.dtype, "scatter_nd");
    if (data.is_scalar() || idx.is_scalar() || upd.is_scalar()) raise(RMLK_ERR_INVALID_ARG, "scalar inputs are not allowed");
    if (idx.dtype != RMLK_I64) unsupported_dtype(idx.dtype, "scatter_nd indices");
    if (upd.dtype != data.dtype) raise(RMLK_ERR_INVALID_ARG, "scatter_nd: updates data type differs from data");
    int red = RMLK_SCATTER_NONE;
    if (const Attr* a = c.attr("reduction")) {
        if (a->kind != Attr::STRING) raise(RMLK_ERR_INVALID_ARG, "scatter_nd: `reduction` must be a string");
        const std::string& s = a->s;
        if (s == "none" || s == "None") red = RMLK_SCATTER_NONE;
        else if (s == "add" || s == "Add") red = RMLK_SCATTER_ADD;
        else if (s == "mul" || s == "Mul") red = RMLK_SCATTER_MUL;
        else if (s == "max" || s == "Max") red = RMLK_SCATTER_MAX;
        else if (s == "min" || s == "Min") red = RMLK_SCATTER_MIN;
        else raise(RMLK_ERR_INVALID_ARG, "unknown value `" + s + "` for `reduction`");
    }
    const size_t ir = idx.shape.size();
    const int64_t k = ir > 1 ? idx.shape[ir - 1] : 1;
    const int64_t n_tuples = ir > 1 ? prod(idx.shape, 0, ir - 1) : prod(idx.shape);
    if (k < 1 || k > static_cast<int64_t>(data.shape.size())) raise(RMLK_ERR_INVALID_ARG, "scatter_nd: index tuple longer than the data rank");
    const int64_t slice_len = prod(data.shape, static_cast<size_t>(k));
    if (upd.numel() != n_tuples * slice_len) raise(RMLK_ERR_INVALID_ARG, "scatter_nd: updates shape does not match indices and data");
    Tensor& o = c.make(0, data.dtype, data.shape);
    check_rc(rmlk_b200_scatter_nd(c.stream(), red, data.dtype, static_cast<int>(data.shape.size()), data.shape.data(), n_tuples, static_cast<int>(k),
                                  data.data, idx.data, upd.data, o.data, static_cast<int*>(c.I.status_word.ptr)));
    c.launched(2);
}

// backend/slice.rs:49-464
void op_slice(const Ctx& c) {
    Tensor& x = c.req(0);
    Tensor& starts = c.req(1);
    Tensor& ends = c.req(2);
    Tensor* axes = c.in(3);
    Tensor* steps = c.in(4);
    if (starts.dtype != ends.dtype) raise(RMLK_ERR_INVALID_ARG, "StartAndEndDataTypeMismatch");
    if (!in_set(x.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64}) || !in_set(starts.dtype, {RMLK_I32, RMLK_I64}))
        unsupported_dtype(x.dtype, "slice");
    const int rank = static_cast<int>(x.shape.size());
    if (rank < 1 || rank > RMLK_MAX_RANK) raise(RMLK_ERR_INVALID_ARG, "slice: rank must be in [1, 8]");
    const std::vector<int64_t> sv = c.I.host_i64(starts), ev = c.I.host_i64(ends);
    std::vector<int64_t> av, pv;
    if (axes) av = c.I.host_i64(*axes);
    if (steps) pv = c.I.host_i64(*steps);
    if (sv.size() != ev.size()) raise(RMLK_ERR_INVALID_ARG, "slice: starts and ends differ in length");
    if (axes && av.size() != sv.size()) raise(RMLK_ERR_INVALID_ARG, "slice: axes and starts differ in length");
    if (steps && pv.size() != (axes ? av.size() : sv.size())) raise(RMLK_ERR_INVALID_ARG, "StepsAndAxesLengthMismatch");
    // i32 index tensors: the reference clamps in i32; sentinels INT_MIN / INT_MAX behave the same in i64.
    int64_t ost[RMLK_MAX_RANK], osp[RMLK_MAX_RANK], osh[RMLK_MAX_RANK];
    check_rc(rmlk_b200_slice_params(rank, x.shape.data(), static_cast<int>(sv.size()), sv.data(), ev.data(), axes ? av.data() : nullptr,
                                    steps ? pv.data() : nullptr, ost, osp, osh));
    Shape oshape(osh, osh + rank);
    Tensor& o = c.make(0, x.dtype, oshape);
    if (o.numel() == 0) return;
    check_rc(rmlk_b200_slice(c.stream(), static_cast<int>(dtype_size_of(x.dtype)), rank, x.shape.data(), osh, ost, osp, x.data, o.data));
    c.launched();
    if (small_mirrored(x) && rank == 1 && x.dtype != RMLK_F16) {
        const bool isf = is_float_dtype(x.dtype);
        std::vector<int64_t> ri;
        std::vector<double> rf;
        for (int64_t i = 0; i < osh[0]; i++) {
            const int64_t s = ost[0] + osp[0] * i;
            if (isf) rf.push_back(x.mf[s]); else ri.push_back(x.mi[s]);
        }
        if (isf) set_mirror_f(o, rf); else set_mirror_i(o, ri);
    }
}

// backend/transpose.rs:44-178
void op_transpose(const Ctx& c) {
    Tensor* xr = c.raw(0);
    if (!xr) raise(RMLK_ERR_INVALID_ARG, "missing input 0");
    if (!in_set(xr->dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64})) unsupported_dtype(xr->dtype, "transpose");
    // Large tensors that stay inside the graph are permuted as a view; the copy happens when (and if) a
    // consumer needs dense data, together with any Expand / Transpose deferred before it.
    if (c.may_defer(0) && xr->numel() > HOST_MIRROR_MAX && xr->shape.size() <= RMLK_MAX_RANK) {
        const int rank = static_cast<int>(xr->shape.size());
        std::vector<int64_t> perm;
        const Attr* a = c.attr("perm");
        bool ok = true;
        if (a) {
            ok = a->kind == Attr::INTS && static_cast<int>(a->ints.size()) == rank;
            if (ok) perm = a->ints;
            std::vector<char> seen(rank, 0);
            for (size_t i = 0; ok && i < perm.size(); i++) {
                ok = perm[i] >= 0 && perm[i] < rank && !seen[perm[i]];
                if (ok) seen[perm[i]] = 1;
            }
        } else {
            for (int i = rank - 1; i >= 0; i--) perm.push_back(i);
        }
        Shape ps, pst;
        std::vector<std::pair<int, int>> groups;
        if (ok && dims_of(*xr, ps, pst, groups)) {
            Shape oshape(rank), nps, npst;
            for (int d = 0; d < rank; d++) {
                oshape[d] = xr->shape[perm[d]];
                for (int p = groups[perm[d]].first; p < groups[perm[d]].second; p++) push_dim(nps, npst, ps[p], pst[p]);
            }
            if (nps.size() <= RMLK_MAX_RANK) {
                c.defer(0, *xr, oshape, nps, npst);
                return;
            }
        }
    }
    Tensor& x = c.req(0);
    const int rank = static_cast<int>(x.shape.size());
    std::vector<int64_t> perm;
    if (const Attr* a = c.attr("perm")) {
        if (a->kind != Attr::INTS) raise(RMLK_ERR_INVALID_ARG, "transpose: `perm` must be a list of ints");
        perm = a->ints;
        if (static_cast<int>(perm.size()) != rank) raise(RMLK_ERR_INVALID_ARG, "InvalidPermLength");
        for (int64_t p : perm)
            if (p < 0 || p >= rank) raise(RMLK_ERR_INVALID_ARG, "PermIndexOutOfBounds { index: " + std::to_string(p) + " }");
    } else {
        for (int i = rank - 1; i >= 0; i--) perm.push_back(i);
    }
    Shape oshape(rank);
    for (int d = 0; d < rank; d++) oshape[d] = x.shape[perm[d]];
    Tensor& o = c.make(0, x.dtype, oshape);
    if (rank == 0) {
        check_cuda(cudaMemcpyAsync(o.data, x.data, o.nbytes(), cudaMemcpyDeviceToDevice, c.I.stream), "transpose scalar copy");
        c.launched();
        return;
    }
    if (rank > RMLK_MAX_RANK) raise(RMLK_ERR_INVALID_ARG, "transpose: rank must be at most 8");
    if (o.numel() == 0) return;
    check_rc(rmlk_b200_transpose(c.stream(), static_cast<int>(dtype_size_of(x.dtype)), rank, x.shape.data(), perm.data(), x.data, o.data));
    c.launched();
}

// Concat(cache, new rows) whose result is carried to the next run as the cache (a bound output, see Binding): the
// cache lives in one buffer with spare room along the axis, only the new rows are copied in behind the old ones,
// and the result is a strided view of that buffer.  False: conditions not met, the general Concat runs.
struct AppendPlan;
Shape cache_strides(const AppendPlan& ap, const Shape& shape, int64_t cap);
void set_strided(Tensor& t, void* data, const Shape& shape, const Shape& st);

// Geometry of appending `add_shape` rows behind `past` along a binding's axis.
struct AppendPlan {
    int64_t rank = 0, axis = 0, outer = 0, inner = 0, tp = 0, tn = 0, total = 0;
    size_t elem = 0, row = 0;  // row: bytes of one entry along the axis
};

bool append_plan(const Binding& b, const Tensor& past, int add_dtype, const Shape& add_shape, AppendPlan& ap) {
    if (past.dtype != add_dtype || past.shape.size() != add_shape.size() || past.shape.empty()) return false;
    ap.rank = static_cast<int64_t>(past.shape.size());
    ap.axis = b.axis < 0 ? b.axis + ap.rank : b.axis;
    if (ap.axis < 0 || ap.axis >= ap.rank) return false;
    for (int64_t d = 0; d < ap.rank; d++)
        if (d != ap.axis && past.shape[d] != add_shape[d]) return false;
    ap.elem = dtype_size_of(past.dtype);
    ap.outer = prod(past.shape, 0, ap.axis);
    ap.inner = prod(past.shape, ap.axis + 1);
    ap.tp = past.shape[ap.axis];
    ap.tn = add_shape[ap.axis];
    ap.total = ap.tp + ap.tn;
    if (ap.elem == 0 || ap.outer <= 0 || ap.inner <= 0) return false;
    ap.row = static_cast<size_t>(ap.inner) * ap.elem;
    return true;
}

// Makes sure the binding's buffer holds the old rows and has room for the new ones.  Runs once per run and cache:
// the producer of the new rows may reserve their slot before the Concat node comes up.
void append_reserve(Instance& I, Binding& b, Tensor& past, const AppendPlan& ap) {
    if (b.reserved_run == I.run_counter && b.reserved_tp == ap.tp && b.cap >= ap.total) return;
    const bool ours = b.store.ptr && past.data == b.store.ptr && b.cap >= ap.tp;  // the view handed out by the previous run
    if (past.lazy && !ours) I.materialize(past);
    if (!(ours && b.cap >= ap.total)) {
        // first run, a cache fed from outside, or out of room: move to a larger buffer (old rows copied once)
        const int64_t ncap = ap.total + std::max<int64_t>(64, ap.total / 2);
        void* np = nullptr;
        check_cuda(cudaMalloc(&np, std::max<size_t>(static_cast<size_t>(ap.outer) * ncap * ap.row, 256)), "cache cudaMalloc");
        if (ap.tp > 0) {
            const size_t spitch = (ours ? static_cast<size_t>(b.cap) : static_cast<size_t>(ap.tp)) * ap.row;
            check_cuda(cudaMemcpy2DAsync(np, static_cast<size_t>(ncap) * ap.row, past.data, spitch, static_cast<size_t>(ap.tp) * ap.row,
                                         static_cast<size_t>(ap.outer), cudaMemcpyDeviceToDevice, I.stream), "cache move");
            I.launches++;
        }
        if (b.store.ptr) {
            check_cuda(cudaStreamSynchronize(I.stream), "cudaStreamSynchronize");  // the old buffer is still being read
            cudaFree(b.store.ptr);
        }
        b.store.ptr = np;
        b.store.cap = static_cast<size_t>(ap.outer) * ncap * ap.row;
        b.cap = ncap;
        // the old rows now live in the new buffer: later readers of `past` must not follow the freed pointer
        if (past.storage == nullptr) set_strided(past, np, past.shape, cache_strides(ap, past.shape, ncap));
    }
    b.reserved_run = I.run_counter;
    b.reserved_tp = ap.tp;
}

// Element strides, per logical dim, of a tensor of `shape` laid out in the binding's buffer (dims before the axis
// step over `cap` entries, the rest is dense).
Shape cache_strides(const AppendPlan& ap, const Shape& shape, int64_t cap) {
    Shape st(ap.rank, 1);
    for (int64_t d = ap.rank - 2; d >= 0; d--) st[d] = st[d + 1] * (d + 1 == ap.axis ? cap : shape[d + 1]);
    return st;
}

// Turns `t` into a view of `shape` at `data` with the given per-dim element strides (an ordinary dense tensor when
// the strides happen to be the dense ones).
void set_strided(Tensor& t, void* data, const Shape& shape, const Shape& st) {
    t.data = data;
    t.storage = nullptr;
    t.pshape.clear();
    t.pstride.clear();
    for (size_t d = 0; d < shape.size(); d++) push_dim(t.pshape, t.pstride, shape[d], st[d]);
    bool dense = true;
    int64_t expect = 1;
    for (size_t d = t.pshape.size(); d-- > 0 && dense;) {
        dense = t.pstride[d] == expect;
        expect *= t.pshape[d];
    }
    t.lazy = !dense;
    if (dense) {
        t.pshape.clear();
        t.pstride.clear();
    }
}

// For the producer of the rows that node `concat_node` will append to a carried cache: reserves the slot and
// returns where the rows go (pointer + per-dim element strides).  False: that Concat is not an in-place append in
// this run, produce the rows the ordinary way.
bool append_slot_for(Instance& I, int concat_node, int dtype, const Shape& rows_shape, void*& ptr, Shape& strides) {
    if (!I.inplace_append_to) return false;
    const NodeDef& cn = I.g.nodes[concat_node];
    if (cn.outputs.empty() || cn.inputs.size() != 2 || cn.inputs[0] < 0) return false;
    const int bi = I.binding_of_out[cn.outputs[0]];
    if (bi < 0 || !I.bindings[bi].appendable) return false;
    Binding& b = I.bindings[bi];
    Tensor& past = I.values[cn.inputs[0]];
    if (!past.present || past.parts > 1) return false;
    AppendPlan ap;
    if (!append_plan(b, past, dtype, rows_shape, ap) || ap.tn <= 0) return false;
    append_reserve(I, b, past, ap);
    ptr = static_cast<char*>(b.store.ptr) + static_cast<size_t>(ap.tp) * ap.row;
    strides = cache_strides(ap, rows_shape, b.cap);
    return true;
}

bool concat_append(const Ctx& c) {
    if (c.n.outputs.empty() || c.n.inputs.size() != 2) return false;
    const int vid = c.n.outputs[0];
    const int bi = c.I.binding_of_out[vid];
    if (bi < 0 || !c.I.bindings[bi].appendable) return false;
    Binding& b = c.I.bindings[bi];
    Tensor* past = c.raw(0);
    Tensor* add = c.raw(1);
    AppendPlan ap;
    if (!past || !add || !append_plan(b, *past, add->dtype, add->shape, ap)) return false;
    append_reserve(c.I, b, *past, ap);
    if (ap.tn > 0) {
        char* slot = static_cast<char*>(b.store.ptr) + static_cast<size_t>(ap.tp) * ap.row;
        const Shape dst = cache_strides(ap, add->shape, b.cap);
        Tensor placed;
        set_strided(placed, slot, add->shape, dst);
        if (add->data == slot && add->storage == nullptr && add->lazy == placed.lazy && add->pshape == placed.pshape &&
            add->pstride == placed.pstride) {
            // the producer of the rows wrote them into the slot already (append_slot_for)
        } else if (add->lazy) {
            // rows that exist only as a view (a block of columns of a wider MatMul result, permuted): one strided ->
            // strided launch instead of a dense copy followed by the append
            Shape ps, pst;
            std::vector<std::pair<int, int>> groups;
            if (c.I.inplace_append_to && dims_of(*add, ps, pst, groups) && ps.size() <= RMLK_MAX_RANK) {
                Shape ost(ps.size(), 0);
                for (int64_t d = 0; d < ap.rank; d++) {
                    int64_t run = dst[d];
                    for (int p2 = groups[d].second - 1; p2 >= groups[d].first; p2--) {
                        ost[p2] = run;
                        run *= ps[p2];
                    }
                }
                if (ap.elem == 4 && ps.size() <= 5) {
                    // collected with the rotary embeddings of the same layer: one launch for all of them
                    rmlk_batch_job j = {};
                    j.kind = RMLK_BATCH_COPY4;
                    j.rank = static_cast<int>(ps.size());
                    for (size_t d = 0; d < 5; d++) {
                        j.shape[d] = d < ps.size() ? ps[d] : 1;
                        j.in_strides[d] = d < ps.size() ? pst[d] : 0;
                        j.out_strides[d] = d < ps.size() ? ost[d] : 0;
                    }
                    j.in = add->data;
                    j.out = slot;
                    c.I.defer_job(j);
                } else {
                    check_rc(rmlk_b200_strided_copy_to(c.stream(), static_cast<int>(ap.elem), static_cast<int>(ps.size()), ps.data(), pst.data(), ost.data(),
                                                       add->data, slot));
                    c.launched();
                }
            } else {
                c.I.materialize(*add);
            }
        }
        if (!add->lazy && add->data != slot) {
            check_cuda(cudaMemcpy2DAsync(slot, static_cast<size_t>(b.cap) * ap.row, add->data, static_cast<size_t>(ap.tn) * ap.row,
                                         static_cast<size_t>(ap.tn) * ap.row, static_cast<size_t>(ap.outer), cudaMemcpyDeviceToDevice, c.I.stream),
                       "cache append");
            c.launched();
        }
    }
    Tensor& o = c.out(0);
    o.dtype = past->dtype;
    o.shape = past->shape;
    o.shape[ap.axis] = ap.total;
    o.mirror_valid = false;
    o.mi.clear();
    o.mf.clear();
    o.parts = 0;
    set_strided(o, b.store.ptr, o.shape, cache_strides(ap, o.shape, b.cap));
    o.present = true;
    return true;
}

// backend/concat.rs:28-198
void op_concat(const Ctx& c) {
    if (concat_append(c)) return;
    Tensor& first = c.req(0);
    if (!in_set(first.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_U32, RMLK_I64, RMLK_U64})) unsupported_dtype(first.dtype, "concat");
    if (first.is_scalar()) raise(RMLK_ERR_INVALID_ARG, "scalars are not allowed");
    const Attr* ax = c.attr("axis");
    if (!ax || ax->kind != Attr::INT) raise(RMLK_ERR_INVALID_ARG, "`axis` is missing");
    const int64_t rank = static_cast<int64_t>(first.shape.size());
    const int64_t axis = normalize_index(ax->i, rank);
    if (axis >= rank) raise(RMLK_ERR_INVALID_ARG, "axis out of bound " + std::to_string(ax->i));
    std::vector<const void*> ptrs;
    std::vector<int64_t> dims;
    std::vector<Tensor*> ins;
    Shape oshape = first.shape;
    int64_t total = 0;
    for (size_t i = 0; i < c.n.inputs.size(); i++) {
        Tensor* t = c.in(i);
        if (!t) break;
        if (static_cast<int64_t>(t->shape.size()) != rank)
            raise(RMLK_ERR_INVALID_ARG, "ShapeMismatch { index: " + std::to_string(i) + ", base_rank: " + std::to_string(rank) + ", found_rank: " + std::to_string(t->shape.size()) + " }");
        if (t->dtype != first.dtype) raise(RMLK_ERR_INVALID_ARG, "concat: input data types differ");
        for (int64_t d = 0; d < rank; d++)
            if (d != axis && t->shape[d] != first.shape[d])
                raise(RMLK_ERR_INVALID_ARG, "DimensionMismatch { axis: " + std::to_string(d) + ", dim: " + std::to_string(t->shape[d]) + ", expected_dim: " + std::to_string(first.shape[d]) + " }");
        total += t->shape[axis];
        ptrs.push_back(t->data);
        dims.push_back(t->shape[axis]);
        ins.push_back(t);
    }
    oshape[axis] = total;
    Tensor& o = c.make(0, first.dtype, oshape);
    if (o.numel() == 0) return;
    check_rc(rmlk_b200_concat(c.stream(), static_cast<int>(dtype_size_of(first.dtype)), static_cast<int>(ptrs.size()), prod(first.shape, 0, axis),
                              prod(first.shape, axis + 1), dims.data(), ptrs.data(), o.data));
    c.launched();
    bool all = rank == 1 && first.dtype != RMLK_F16 && o.numel() <= HOST_MIRROR_MAX;
    for (Tensor* t : ins) all = all && small_mirrored(*t);
    if (all) {
        if (is_float_dtype(first.dtype)) {
            std::vector<double> r;
            for (Tensor* t : ins) r.insert(r.end(), t->mf.begin(), t->mf.end());
            set_mirror_f(o, r);
        } else {
            std::vector<int64_t> r;
            for (Tensor* t : ins) r.insert(r.end(), t->mi.begin(), t->mi.end());
            set_mirror_i(o, r);
        }
    }
}

// backend/expand.rs:49-216
void op_expand(const Ctx& c) {
    Tensor* xr = c.raw(0);
    if (!xr) raise(RMLK_ERR_INVALID_ARG, "missing input 0");
    Tensor& sh = c.req(1);
    if (!in_set(xr->dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_U32, RMLK_I64, RMLK_U64})) unsupported_dtype(xr->dtype, "expand");
    if (sh.dtype != RMLK_I64) unsupported_dtype(sh.dtype, "expand shape");
    const std::vector<int64_t> target = c.I.host_i64(sh);
    for (int64_t v : target)
        if (v < 0) raise(RMLK_ERR_INVALID_ARG, "expand: negative dimension in shape");
    Shape oshape;
    if (!broadcast_shape(xr->shape, target, oshape))
        raise(RMLK_ERR_INVALID_ARG, "incompatible shapes for broadcast: " + shape_str(xr->shape) + " " + shape_str(target));
    if (oshape.size() > RMLK_MAX_RANK) raise(RMLK_ERR_INVALID_ARG, "expand: rank must be at most 8");
    // Large results that stay inside the graph are broadcast as a view (stride 0 along the repeated dims).
    if (c.may_defer(0) && prod(oshape) > HOST_MIRROR_MAX && xr->numel() > 0) {
        Shape ps, pst, nps, npst;
        std::vector<std::pair<int, int>> groups;
        if (dims_of(*xr, ps, pst, groups)) {
            const size_t orank = oshape.size(), xrank = xr->shape.size();
            for (size_t d = 0; d < orank; d++) {
                if (d + xrank < orank) {
                    push_dim(nps, npst, oshape[d], 0);
                    continue;
                }
                const size_t j = d - (orank - xrank);
                if (xr->shape[j] == oshape[d]) {
                    for (int p = groups[j].first; p < groups[j].second; p++) push_dim(nps, npst, ps[p], pst[p]);
                } else {
                    push_dim(nps, npst, oshape[d], 0);
                }
            }
            if (nps.size() <= RMLK_MAX_RANK) {
                c.defer(0, *xr, oshape, nps, npst);
                return;
            }
        }
    }
    Tensor& x = c.req(0);
    Tensor& o = c.make(0, x.dtype, oshape);
    if (o.numel() == 0) return;
    const Shape ish = kshape(x);
    const Shape ks = oshape.empty() ? Shape{1} : oshape;
    check_rc(rmlk_b200_expand(c.stream(), static_cast<int>(dtype_size_of(x.dtype)), static_cast<int>(ish.size()), ish.data(), static_cast<int>(ks.size()),
                              ks.data(), x.data, o.data));
    c.launched();
    if (small_mirrored(x) && o.numel() <= HOST_MIRROR_MAX && x.dtype != RMLK_F16) {
        const int64_t n = o.numel();
        if (is_float_dtype(x.dtype)) {
            std::vector<double> r(n);
            for (int64_t i = 0; i < n; i++) r[i] = x.mf[bindex(x.shape, oshape, i)];
            set_mirror_f(o, r);
        } else {
            std::vector<int64_t> r(n);
            for (int64_t i = 0; i < n; i++) r[i] = x.mi[bindex(x.shape, oshape, i)];
            set_mirror_i(o, r);
        }
    }
}

// backend/trilu.rs:48-146
void op_trilu(const Ctx& c) {
    Tensor& x = c.req(0);
    if (!in_set(x.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_U32, RMLK_I64, RMLK_U64})) unsupported_dtype(x.dtype, "trilu");
    const bool upper = c.attr_int("upper", 1) != 0;
    int64_t k = 0;
    if (Tensor* kt = c.in(1)) {
        if (!kt->is_scalar()) raise(RMLK_ERR_INVALID_ARG, "InvalidKTensor");
        if (kt->dtype != RMLK_I64) unsupported_dtype(kt->dtype, "trilu k");
        k = c.I.host_i64(*kt)[0];
    }
    Tensor& o = c.make(0, x.dtype, x.shape);
    if (o.numel() == 0) return;
    // [batch, R, C] view: runtime/src/utils/mod.rs:226-239
    int64_t b = 1, r = 1, cc = 1;
    const size_t rank = x.shape.size();
    if (rank == 1) cc = x.shape[0];
    else if (rank >= 2) { r = x.shape[rank - 2]; cc = x.shape[rank - 1]; b = prod(x.shape, 0, rank - 2); }
    check_rc(rmlk_b200_trilu(c.stream(), static_cast<int>(dtype_size_of(x.dtype)), b, r, cc, upper ? 1 : 0, k, x.data, o.data));
    c.launched();
}

// backend/range.rs:28-205
void op_range(const Ctx& c) {
    Tensor& s = c.req(0);
    Tensor& l = c.req(1);
    Tensor& d = c.req(2);
    if (!in_set(s.dtype, {RMLK_F16, RMLK_F32, RMLK_F64, RMLK_I32, RMLK_I64})) unsupported_dtype(s.dtype, "range");
    if (l.dtype != s.dtype || d.dtype != s.dtype) raise(RMLK_ERR_INVALID_ARG, "range: start, limit and delta must share a data type");
    if (s.numel() != 1 || l.numel() != 1 || d.numel() != 1) raise(RMLK_ERR_INVALID_ARG, "range: inputs must be scalars");
    int64_t count = 0;
    union { int32_t i32; int64_t i64; float f32; double f64; uint16_t f16; } sv{}, dv{};
    if (is_int_dtype(s.dtype)) {
        const int64_t start = c.I.host_i64(s)[0], limit = c.I.host_i64(l)[0], delta = c.I.host_i64(d)[0];
        if (delta == 0) raise(RMLK_ERR_INVALID_ARG, "range: delta must not be zero");
        count = std::max<int64_t>((limit - start) / delta, 0);  // truncating division (range.rs:140-152)
        if (s.dtype == RMLK_I32) { sv.i32 = static_cast<int32_t>(start); dv.i32 = static_cast<int32_t>(delta); }
        else { sv.i64 = start; dv.i64 = delta; }
    } else {
        if (s.dtype == RMLK_F16) unsupported_dtype(s.dtype, "range (f16 scalars are not mirrored on the host)");
        const double start = c.I.host_f64(s)[0], limit = c.I.host_f64(l)[0], delta = c.I.host_f64(d)[0];
        double cnt;
        if (s.dtype == RMLK_F32) {
            cnt = std::ceil((static_cast<float>(limit) - static_cast<float>(start)) / static_cast<float>(delta));
            sv.f32 = static_cast<float>(start);
            dv.f32 = static_cast<float>(delta);
        } else {
            cnt = std::ceil((limit - start) / delta);
            sv.f64 = start;
            dv.f64 = delta;
        }
        if (!(cnt >= 0.0) || cnt > 9.0e15) raise(RMLK_ERR_INVALID_ARG, "ConversionError");
        count = static_cast<int64_t>(cnt);
    }
    Tensor& o = c.make(0, s.dtype, Shape{count});
    if (count == 0) return;
    check_rc(rmlk_b200_range(c.stream(), s.dtype, count, &sv, &dv, o.data));
    c.launched();
    if (count <= HOST_MIRROR_MAX) {
        if (is_int_dtype(s.dtype)) {
            std::vector<int64_t> r(count);
            const int64_t st = s.dtype == RMLK_I32 ? sv.i32 : sv.i64, de = s.dtype == RMLK_I32 ? dv.i32 : dv.i64;
            for (int64_t i = 0; i < count; i++) r[i] = wrap_int(s.dtype, st + i * de);
            set_mirror_i(o, r);
        } else {
            std::vector<double> r(count);
            for (int64_t i = 0; i < count; i++) {
                if (s.dtype == RMLK_F32) {
                    const float pr = static_cast<float>(i) * dv.f32;
                    r[i] = static_cast<double>(sv.f32 + pr);
                } else {
                    r[i] = sv.f64 + static_cast<double>(i) * dv.f64;
                }
            }
            set_mirror_f(o, r);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// shape-only ops: metadata changes, no payload copies
// ---------------------------------------------------------------------------------------------
// backend/reshape.rs:60-160
void op_reshape(const Ctx& c) {
    // a deferred view keeps its element order under Reshape, so it can stay deferred
    Tensor& x = c.may_defer(0) && c.raw(0) ? *c.raw(0) : c.req(0);
    Tensor& sh = c.req(1);
    if (sh.dtype != RMLK_I64) unsupported_dtype(sh.dtype, "reshape shape");
    const bool allow_zero = c.attr_int("allowzero", 0) != 0;
    std::vector<int64_t> dims = sh.shape.empty() ? std::vector<int64_t>{} : c.I.host_i64(sh);
    Shape target(dims.size(), 0);
    int neg = -1;
    bool has_zero = false;
    for (size_t i = 0; i < dims.size(); i++) {
        if (dims[i] == -1) {
            if (neg >= 0 || (allow_zero && has_zero)) raise(RMLK_ERR_INVALID_ARG, "ZeroDim and negative dimensions are not allowed");
            neg = static_cast<int>(i);
            target[i] = 1;
        } else if (dims[i] == 0) {
            if (allow_zero && neg >= 0) raise(RMLK_ERR_INVALID_ARG, "ZeroDim and negative dimensions are not allowed");
            has_zero = true;
            if (!allow_zero) {
                if (i >= x.shape.size()) raise(RMLK_ERR_INVALID_ARG, "index out of range");
                target[i] = x.shape[i];
            }
        } else if (dims[i] < 0) {
            raise(RMLK_ERR_INVALID_ARG, "invalid index");
        } else {
            target[i] = dims[i];
        }
    }
    const int64_t total = x.numel();
    if (neg >= 0) {
        const int64_t cur = prod(target);
        if (cur == 0) {
            if (total != 0) raise(RMLK_ERR_INVALID_ARG, "unable to hold the same number of elements");
        } else {
            if (total % cur != 0) raise(RMLK_ERR_INVALID_ARG, "unable to hold the same number of elements");
            target[neg] = total / cur;
        }
    }
    if (prod(target) != total) raise(RMLK_ERR_INVALID_ARG, "unable to hold the same number of elements");
    c.view(0, x, target);
}

// backend/unsqueeze.rs:60-130
void op_unsqueeze(const Ctx& c) {
    // inserting size-1 dims does not change the element order: a deferred view stays deferred
    Tensor& x = c.may_defer(0) && c.raw(0) ? *c.raw(0) : c.req(0);
    std::vector<int64_t> axes;
    if (Tensor* at = c.in(1)) {
        if (at->shape.size() != 1) raise(RMLK_ERR_INVALID_ARG, "InvalidAxesRank");
        axes = c.I.host_i64(*at);
    } else if (const Attr* a = c.attr("axes")) {
        axes = a->ints;
    } else {
        raise(RMLK_ERR_INVALID_ARG, "unsqueeze: missing axes");
    }
    for (size_t i = 0; i < axes.size(); i++)
        for (size_t j = i + 1; j < axes.size(); j++)
            if (axes[i] == axes[j]) raise(RMLK_ERR_INVALID_ARG, "DuplicateAxes");
    const int64_t erank = static_cast<int64_t>(axes.size() + x.shape.size());
    Shape oshape(erank, 0);
    for (int64_t a : axes) {
        const int64_t n = normalize_index(a, erank);
        if (n >= erank) raise(RMLK_ERR_INVALID_ARG, "axis out of bound " + std::to_string(a));
        oshape[n] = -1;
    }
    size_t src = 0;
    for (int64_t i = 0; i < erank; i++) {
        if (oshape[i] == -1) oshape[i] = 1;
        else oshape[i] = x.shape[src++];
    }
    c.view(0, x, oshape);
}

// runtime/src/providers/cpu/flatten.rs
void op_flatten(const Ctx& c) {
    Tensor& x = c.may_defer(0) && c.raw(0) ? *c.raw(0) : c.req(0);
    const int64_t rank = static_cast<int64_t>(x.shape.size());
    int64_t axis = c.attr_int("axis", 1);
    if (axis < 0) axis += rank;
    if (axis < 0 || axis > rank) raise(RMLK_ERR_INVALID_ARG, "flatten: axis out of range");
    c.view(0, x, Shape{prod(x.shape, 0, axis), prod(x.shape, axis)});
}

void store_small_i64(const Ctx& c, Tensor& o, const std::vector<int64_t>& vals) {
    // values travel as kernel parameters; larger tensors go through an async copy from the mirror
    const int64_t n = static_cast<int64_t>(vals.size());
    for (int64_t b = 0; b < n; b += 32) {
        const int cnt = static_cast<int>(std::min<int64_t>(32, n - b));
        check_rc(rmlk_b200_store_small(c.stream(), cnt, reinterpret_cast<const uint64_t*>(vals.data() + b), static_cast<int64_t*>(o.data) + b));
        c.launched();
    }
}

// backend/shape.rs:30-80
void op_shape(const Ctx& c) {
    Tensor* xr = c.raw(0);  // only the dims are read: a deferred view stays deferred
    if (!xr) raise(RMLK_ERR_INVALID_ARG, "missing input 0");
    Tensor& x = *xr;
    const int64_t rank = static_cast<int64_t>(x.shape.size());
    int64_t start = c.attr_int("start", 0), end = c.attr_int("end", rank);
    if (start < 0) start += rank;
    if (end < 0) end += rank;
    start = std::min(std::max<int64_t>(start, 0), rank);
    end = std::min(std::max<int64_t>(end, 0), rank);
    std::vector<int64_t> vals;
    for (int64_t i = start; i < end; i++) vals.push_back(x.shape[i]);
    Tensor& o = c.make(0, RMLK_I64, Shape{static_cast<int64_t>(vals.size())});
    store_small_i64(c, o, vals);
    set_mirror_i(o, vals);
}

// backend/constant_of_shape.rs:30-70
void op_constant_of_shape(const Ctx& c) {
    Tensor& sh = c.req(0);
    if (sh.dtype != RMLK_I64) unsupported_dtype(sh.dtype, "constant_of_shape shape");
    const std::vector<int64_t> dims = c.I.host_i64(sh);
    for (int64_t v : dims)
        if (v < 0) raise(RMLK_ERR_INVALID_ARG, "constant_of_shape: negative dimension");
    int dtype = RMLK_F32;
    uint8_t value[8] = {0};
    if (const Attr* a = c.attr("value")) {
        if (a->kind != Attr::TENSOR || a->t_data.size() < dtype_size_of(a->t_dtype) || dtype_size_of(a->t_dtype) == 0)
            raise(RMLK_ERR_INVALID_ARG, "constant_of_shape: `value` must be a one-element tensor");
        dtype = a->t_dtype;
        std::memcpy(value, a->t_data.data(), dtype_size_of(dtype));
    }
    Tensor& o = c.make(0, dtype, dims);
    if (o.numel() == 0) return;
    check_rc(rmlk_b200_fill(c.stream(), static_cast<int>(dtype_size_of(dtype)), o.numel(), value, o.data));
    c.launched();
    if (o.numel() <= HOST_MIRROR_MAX && dtype != RMLK_F16) {
        if (is_float_dtype(dtype)) {
            double v = 0;
            if (dtype == RMLK_F32) { float f; std::memcpy(&f, value, 4); v = f; } else std::memcpy(&v, value, 8);
            set_mirror_f(o, std::vector<double>(o.numel(), v));
        } else {
            int64_t v = 0;
            switch (dtype_size_of(dtype)) {
                case 1: v = dtype == RMLK_I8 ? static_cast<int8_t>(value[0]) : value[0]; break;
                case 2: { int16_t t; std::memcpy(&t, value, 2); v = dtype == RMLK_I16 ? t : static_cast<uint16_t>(t); break; }
                case 4: { int32_t t; std::memcpy(&t, value, 4); v = dtype == RMLK_I32 ? t : static_cast<uint32_t>(t); break; }
                default: std::memcpy(&v, value, 8); break;
            }
            set_mirror_i(o, std::vector<int64_t>(o.numel(), v));
        }
    }
}

}  // namespace

size_t dtype_size_of(int dt) { return rmlk_b200_dtype_size(dt); }

// ---------------------------------------------------------------------------------------------
// fused chains
// ---------------------------------------------------------------------------------------------
namespace {

struct Matcher {
    const Graph& g;
    std::vector<int> producer, uses;
    const std::vector<int>& group_of_node;
    Matcher(const Graph& gr, const std::vector<int>& gon) : g(gr), producer(gr.values.size(), -1), uses(gr.values.size(), 0), group_of_node(gon) {
        for (size_t i = 0; i < g.nodes.size(); i++) {
            for (int v : g.nodes[i].outputs)
                if (v >= 0) producer[v] = static_cast<int>(i);
            for (int v : g.nodes[i].inputs)
                if (v >= 0) uses[v]++;
        }
    }
    // node producing `v` if it has the given op, `v` feeds exactly one node and never leaves the graph
    int inner(int v, int op) const {
        if (v < 0) return -1;
        const int p = producer[v];
        if (p < 0 || g.nodes[p].op != op || group_of_node[p] >= 0) return -1;
        const ValueDef& d = g.values[v];
        if (uses[v] != 1 || d.is_output || d.is_input || d.is_const) return -1;
        return p;
    }
    bool is_const(int v) const { return v >= 0 && g.values[v].is_const; }
    int in(int node, size_t i) const { return i < g.nodes[node].inputs.size() ? g.nodes[node].inputs[i] : -1; }
    size_t n_in(int node) const {
        size_t n = g.nodes[node].inputs.size();
        while (n > 0 && g.nodes[node].inputs[n - 1] < 0) n--;
        return n;
    }
};

bool scalar_f32(const Tensor& t, float& v) {
    if (t.dtype != RMLK_F32 || t.numel() != 1 || !t.mirror_valid || t.mf.empty()) return false;
    v = static_cast<float>(t.mf[0]);
    return true;
}

// Element strides of `t` (dense) when broadcast to `shape` (same rank or lower, right-aligned); false if not broadcastable.
bool bcast_strides(const Tensor& t, const Shape& shape, int64_t* out) {
    if (t.shape.size() > shape.size()) return false;
    const Shape st = dense_strides(t.shape);
    const size_t lead = shape.size() - t.shape.size();
    for (size_t d = 0; d < shape.size(); d++) {
        if (d < lead) {
            out[d] = 0;
            continue;
        }
        const int64_t n = t.shape[d - lead];
        if (n == shape[d]) out[d] = n == 1 ? 0 : st[d - lead];
        else if (n == 1) out[d] = 0;
        else return false;
    }
    return true;
}

}  // namespace

void Instance::find_fusions() {
    group_of_node.assign(g.nodes.size(), -1);
    groups.clear();
    parts_ok_value.assign(g.values.size(), 0);
    append_consumer.assign(g.values.size(), -1);
    if (!fusion) return;
    Matcher m(g, group_of_node);
    for (size_t i = 0; i < g.nodes.size(); i++) {
        const NodeDef& n = g.nodes[i];
        if (n.op != RMLK_OP_CONCAT || m.n_in(static_cast<int>(i)) != 2) continue;
        const int v = n.inputs[1];
        const ValueDef& d = g.values[v];
        if (v >= 0 && m.uses[v] == 1 && !d.is_output && !d.is_input && !d.is_const) append_consumer[v] = static_cast<int>(i);
    }
    auto commit = [&](FusedGroup& fg) {
        std::sort(fg.members.begin(), fg.members.end());
        fg.root = fg.members.back();
        for (int n : fg.members) group_of_node[n] = static_cast<int>(groups.size());
        groups.push_back(fg);
    };
    for (size_t r = 0; r < g.nodes.size(); r++) {
        const NodeDef& root = g.nodes[r];
        if (group_of_node[r] >= 0) continue;
        const int ri = static_cast<int>(r);
        if (root.op == RMLK_OP_MUL && m.n_in(ri) == 2) {
            bool done = false;
            for (int side = 0; side < 2 && !done; side++) {
                // RMSNorm: Mul(Div(x, Sqrt(Add(ReduceMean(Pow(x, c)), eps))), w)
                const int dv = m.in(ri, side), w = m.in(ri, 1 - side);
                const int n_div = m.inner(dv, RMLK_OP_DIV);
                if (n_div >= 0) {
                    const int x = m.in(n_div, 0), n_sqrt = m.inner(m.in(n_div, 1), RMLK_OP_SQRT);
                    const int n_add = n_sqrt >= 0 ? m.inner(m.in(n_sqrt, 0), RMLK_OP_ADD) : -1;
                    for (int s2 = 0; s2 < 2 && n_add >= 0 && !done; s2++) {
                        const int var = m.in(n_add, s2), eps = m.in(n_add, 1 - s2);
                        const int n_mean = m.inner(var, RMLK_OP_REDUCE_MEAN);
                        if (n_mean < 0 || !m.is_const(eps) || m.n_in(n_mean) != 1) continue;
                        const NodeDef& mean = g.nodes[n_mean];
                        auto ax = mean.attrs.find("axes");
                        auto kd = mean.attrs.find("keepdims");
                        if (ax == mean.attrs.end() || ax->second.kind != Attr::INTS || ax->second.ints.size() != 1 || ax->second.ints[0] != -1) continue;
                        if (kd != mean.attrs.end() && kd->second.i != 1) continue;
                        const int n_pow = m.inner(m.in(n_mean, 0), RMLK_OP_POW);
                        if (n_pow < 0 || m.in(n_pow, 0) != x || !m.is_const(m.in(n_pow, 1))) continue;
                        FusedGroup fg;
                        fg.kind = FusedGroup::RMSNORM;
                        fg.members = {n_pow, n_mean, n_add, n_sqrt, n_div, ri};
                        fg.v[0] = x; fg.v[1] = w; fg.v[2] = eps; fg.v[3] = m.in(n_pow, 1);
                        // x = Add(a, b) made just for this chain and for readers that come after it (the residual
                        // stream of a decoder layer): the Add joins the chain, whose kernel then writes x as well
                        const int n_res = x >= 0 ? m.producer[x] : -1;
                        const ValueDef* xd = x >= 0 ? &g.values[x] : nullptr;
                        if (add_norm && n_res >= 0 && g.nodes[n_res].op == RMLK_OP_ADD && group_of_node[n_res] < 0 && m.n_in(n_res) == 2 &&
                            !xd->is_output && !xd->is_input && !xd->is_const) {
                            bool later = true;
                            for (size_t j = 0; j < g.nodes.size() && later; j++) {
                                const int ji = static_cast<int>(j);
                                if (ji > ri || ji == n_res || std::find(fg.members.begin(), fg.members.end(), ji) != fg.members.end()) continue;
                                for (int v : g.nodes[j].inputs) later = later && v != x;
                            }
                            if (later) {
                                int a_in = m.in(n_res, 0), b_in = m.in(n_res, 1);
                                auto sole_matmul = [&](int v) {
                                    const int pn = v >= 0 ? m.producer[v] : -1;
                                    return pn >= 0 && g.nodes[pn].op == RMLK_OP_MATMUL && m.uses[v] == 1 && !g.values[v].is_output;
                                };
                                if (!sole_matmul(b_in) && sole_matmul(a_in)) std::swap(a_in, b_in);
                                if (sole_matmul(b_in)) parts_ok_value[b_in] = 1;
                                fg.members.push_back(n_res);
                                fg.v[4] = a_in; fg.v[5] = b_in;
                            }
                        }
                        commit(fg);
                        done = true;
                    }
                }
                if (done) break;
                // SwiGLU gate: Mul(Mul(g, Sigmoid(g)), u)
                const int n_silu = m.inner(m.in(ri, side), RMLK_OP_MUL);
                if (n_silu >= 0 && m.n_in(n_silu) == 2) {
                    for (int s2 = 0; s2 < 2 && !done; s2++) {
                        const int gate = m.in(n_silu, s2), n_sig = m.inner(m.in(n_silu, 1 - s2), RMLK_OP_SIGMOID);
                        if (n_sig < 0 || m.in(n_sig, 0) != gate) continue;
                        FusedGroup fg;
                        fg.kind = FusedGroup::SWIGLU;
                        fg.members = {n_sig, n_silu, ri};
                        fg.v[0] = gate; fg.v[1] = m.in(ri, 1 - side);
                        commit(fg);
                        done = true;
                    }
                }
            }
        } else if (root.op == RMLK_OP_ADD && m.n_in(ri) == 2) {
            // rotary embedding: Add(Mul(x, cos), Mul(Concat(Neg(Slice(x, hi)), Slice(x, lo)), sin))
            bool done = false;
            for (int side = 0; side < 2 && !done; side++) {
                const int n_xc = m.inner(m.in(ri, side), RMLK_OP_MUL), n_xs = m.inner(m.in(ri, 1 - side), RMLK_OP_MUL);
                if (n_xc < 0 || n_xs < 0 || n_xc == n_xs || m.n_in(n_xc) != 2 || m.n_in(n_xs) != 2) continue;
                for (int s2 = 0; s2 < 2 && !done; s2++) {
                    const int n_cat = m.inner(m.in(n_xs, s2), RMLK_OP_CONCAT), sinv = m.in(n_xs, 1 - s2);
                    if (n_cat < 0 || m.n_in(n_cat) != 2) continue;
                    const int n_neg = m.inner(m.in(n_cat, 0), RMLK_OP_NEG), n_lo = m.inner(m.in(n_cat, 1), RMLK_OP_SLICE);
                    const int n_hi = n_neg >= 0 ? m.inner(m.in(n_neg, 0), RMLK_OP_SLICE) : -1;
                    if (n_lo < 0 || n_hi < 0 || n_lo == n_hi) continue;
                    const int x = m.in(n_lo, 0);
                    if (m.in(n_hi, 0) != x) continue;
                    bool consts = true;
                    for (int sl : {n_lo, n_hi})
                        for (size_t k = 1; k < m.n_in(sl); k++) consts = consts && m.is_const(m.in(sl, k));
                    if (!consts || m.n_in(n_lo) < 4 || m.n_in(n_hi) < 4) continue;
                    int cosv = -1;
                    if (m.in(n_xc, 0) == x) cosv = m.in(n_xc, 1);
                    else if (m.in(n_xc, 1) == x) cosv = m.in(n_xc, 0);
                    if (cosv < 0) continue;
                    FusedGroup fg;
                    fg.kind = FusedGroup::ROPE;
                    fg.members = {n_xc, n_lo, n_hi, n_neg, n_cat, n_xs, ri};
                    fg.v[0] = x; fg.v[1] = cosv; fg.v[2] = sinv; fg.v[3] = n_lo; fg.v[4] = n_hi; fg.v[5] = n_cat;  // v[3..5]: node ids
                    commit(fg);
                    done = true;
                }
            }
        } else if ((root.op == RMLK_OP_COS || root.op == RMLK_OP_SIN) && m.n_in(ri) == 1) {
            // rotary tables: Cos(emb) and Sin(emb) with emb = Concat(f, f) on the last axis and f = Mul(a, b); the later of the
            // two nodes is the root and both outputs are written there
            const int emb = m.in(ri, 0);
            const int n_cat = emb >= 0 ? m.producer[emb] : -1;
            if (n_cat < 0 || g.nodes[n_cat].op != RMLK_OP_CONCAT || group_of_node[n_cat] >= 0 || m.n_in(n_cat) != 2 || m.uses[emb] != 2 ||
                g.values[emb].is_output)
                continue;
            const int f = m.in(n_cat, 0);
            if (f < 0 || m.in(n_cat, 1) != f || m.uses[f] != 2 || g.values[f].is_output) continue;
            const int n_mul = m.producer[f];
            if (n_mul < 0 || g.nodes[n_mul].op != RMLK_OP_MUL || group_of_node[n_mul] >= 0 || m.n_in(n_mul) != 2) continue;
            const int64_t cat_axis = Ctx{*this, g.nodes[n_cat]}.attr_int("axis", 0);
            if (cat_axis != -1) continue;
            int partner = -1;
            for (size_t j = 0; j < g.nodes.size() && partner < 0; j++)
                if (static_cast<int>(j) != ri && (g.nodes[j].op == RMLK_OP_COS || g.nodes[j].op == RMLK_OP_SIN) && g.nodes[j].op != root.op &&
                    m.n_in(static_cast<int>(j)) == 1 && m.in(static_cast<int>(j), 0) == emb && group_of_node[j] < 0)
                    partner = static_cast<int>(j);
            if (partner < 0 || partner > ri) continue;  // matched from the later node only
            // nothing may read the earlier node's output before the root has run
            const int early = g.nodes[partner].outputs.empty() ? -1 : g.nodes[partner].outputs[0];
            bool later = early >= 0;
            for (int j = 0; j <= ri && later; j++)
                for (int v : g.nodes[j].inputs) later = later && v != early;
            if (!later) continue;
            FusedGroup fg;
            fg.kind = FusedGroup::ROPE_TABLES;
            fg.members = {n_mul, n_cat, partner, ri};
            fg.v[0] = m.in(n_mul, 0); fg.v[1] = m.in(n_mul, 1);
            fg.v[2] = root.op == RMLK_OP_COS ? ri : partner;   // node ids: Cos, Sin
            fg.v[3] = root.op == RMLK_OP_SIN ? ri : partner;
            commit(fg);
        } else if (root.op == RMLK_OP_WHERE && m.n_in(ri) == 3) {
            // attention mask of an exported decoder:
            //   Where(Unsqueeze(Equal(Cast(attention_mask), c0)), X, Unsqueeze(Where(Equal(Trilu(ConstantOfShape(st), k), c1), Y, Z)))
            const int n_u_pad = m.inner(m.in(ri, 0), RMLK_OP_UNSQUEEZE), n_u_c = m.inner(m.in(ri, 2), RMLK_OP_UNSQUEEZE);
            const int xv = m.in(ri, 1);
            if (n_u_pad < 0 || n_u_c < 0 || !m.is_const(xv)) continue;
            const int n_eq_pad = m.inner(m.in(n_u_pad, 0), RMLK_OP_EQUAL), n_w2 = m.inner(m.in(n_u_c, 0), RMLK_OP_WHERE);
            if (n_eq_pad < 0 || n_w2 < 0 || m.n_in(n_eq_pad) != 2 || m.n_in(n_w2) != 3) continue;
            int n_cast = -1, c0 = -1;
            for (int side = 0; side < 2 && n_cast < 0; side++) {
                const int nc = m.inner(m.in(n_eq_pad, side), RMLK_OP_CAST);
                if (nc >= 0 && m.is_const(m.in(n_eq_pad, 1 - side))) {
                    n_cast = nc;
                    c0 = m.in(n_eq_pad, 1 - side);
                }
            }
            if (n_cast < 0) continue;
            const int n_eq_tri = m.inner(m.in(n_w2, 0), RMLK_OP_EQUAL);
            const int yv = m.in(n_w2, 1), zv = m.in(n_w2, 2);
            if (n_eq_tri < 0 || m.n_in(n_eq_tri) != 2 || !m.is_const(yv) || !m.is_const(zv)) continue;
            int n_tri = -1, c1 = -1;
            for (int side = 0; side < 2 && n_tri < 0; side++) {
                const int nt = m.inner(m.in(n_eq_tri, side), RMLK_OP_TRILU);
                if (nt >= 0 && m.is_const(m.in(n_eq_tri, 1 - side))) {
                    n_tri = nt;
                    c1 = m.in(n_eq_tri, 1 - side);
                }
            }
            if (n_tri < 0) continue;
            const int n_ones = m.inner(m.in(n_tri, 0), RMLK_OP_CONSTANT_OF_SHAPE);
            if (n_ones < 0) continue;
            FusedGroup fg;
            fg.kind = FusedGroup::MASK;
            fg.members = {n_ones, n_tri, n_eq_tri, n_w2, n_u_c, n_cast, n_eq_pad, n_u_pad, ri};
            fg.v[0] = m.in(n_cast, 0); fg.v[1] = m.in(n_ones, 0); fg.v[2] = m.in(n_tri, 1);
            fg.v[3] = c1; fg.v[4] = yv; fg.v[5] = zv; fg.v[6] = c0; fg.v[7] = xv;
            fg.v[8] = n_ones; fg.v[9] = n_tri; fg.v[10] = n_u_c; fg.v[11] = n_u_pad;   // node ids
            commit(fg);
            // (the Cast node id is members[5] before sorting; it is looked up again by op when the chain runs)
        } else if (root.op == RMLK_OP_SOFTMAX) {
            // Softmax(Add(Mul(scores, scale), mask))
            const int n_add = m.inner(m.in(ri, 0), RMLK_OP_ADD);
            bool done = false;
            for (int side = 0; side < 2 && n_add >= 0 && !done; side++) {
                const int n_mul = m.inner(m.in(n_add, side), RMLK_OP_MUL), mask = m.in(n_add, 1 - side);
                if (n_mul < 0 || m.n_in(n_mul) != 2) continue;
                for (int s2 = 0; s2 < 2 && !done; s2++) {
                    const int scores = m.in(n_mul, s2), scale = m.in(n_mul, 1 - s2);
                    if (!m.is_const(scale) || m.is_const(scores)) continue;
                    FusedGroup fg;
                    fg.kind = FusedGroup::SCALE_MASK_SOFTMAX;
                    fg.members = {n_mul, n_add, ri};
                    fg.v[0] = scores; fg.v[1] = scale; fg.v[2] = mask;
                    commit(fg);
                    done = true;
                    // scores = MatMul(q, K^T) read only here, probabilities read only by MatMul(., V): the five nodes
                    // are one attention group (the chain above stays available on its own for runs that do not fit)
                    const int n_sc = m.inner(scores, RMLK_OP_MATMUL);
                    const int probs = root.outputs.empty() ? -1 : root.outputs[0];
                    int n_ctx = -1;
                    if (attention && n_sc >= 0 && probs >= 0 && m.uses[probs] == 1 && !g.values[probs].is_output) {
                        for (size_t j = r + 1; j < g.nodes.size() && n_ctx < 0; j++)
                            if (g.nodes[j].op == RMLK_OP_MATMUL && group_of_node[j] < 0 && m.n_in(static_cast<int>(j)) == 2 && g.nodes[j].inputs[0] == probs)
                                n_ctx = static_cast<int>(j);
                    }
                    if (n_ctx >= 0 && m.n_in(n_sc) == 2) {
                        FusedGroup at;
                        at.kind = FusedGroup::ATTENTION;
                        at.sub = static_cast<int>(groups.size()) - 1;
                        at.members = {n_sc, n_mul, n_add, ri, n_ctx};
                        at.v[0] = m.in(n_sc, 0); at.v[1] = scale; at.v[2] = mask; at.v[3] = m.in(n_sc, 1); at.v[4] = m.in(n_ctx, 1);
                        commit(at);
                    }
                }
            }
        }
    }
    // a skipped member's inputs are read when the root runs: they stay alive until then
    last_use.assign(g.values.size(), -1);
    for (size_t i = 0; i < g.nodes.size(); i++) {
        const int at = group_of_node[i] >= 0 ? groups[group_of_node[i]].root : static_cast<int>(i);
        for (int v : g.nodes[i].inputs)
            if (v >= 0) last_use[v] = std::max(last_use[v], at);
    }
}

// Runs the fused kernel of `fg` if the tensors of this run meet its conditions.  False: nothing was launched and no
// output was touched; the caller runs the member nodes instead.
// a rotary embedding as a collected job (out_strides == nullptr: dense output)
static rmlk_batch_job rope_job(const Shape& oshape, const int64_t* xstr, const int64_t* cstr, const int64_t* sstr, const void* x, const void* cosv,
                               const void* sinv, void* out, const int64_t* out_strides) {
    rmlk_batch_job j = {};
    j.kind = RMLK_BATCH_ROPE;
    j.rank = 4;
    int64_t run = 1;
    for (int d = 3; d >= 0; d--) {
        j.shape[d] = oshape[d];
        j.in_strides[d] = xstr[d];
        j.cos_strides[d] = cstr[d];
        j.sin_strides[d] = sstr[d];
        j.out_strides[d] = out_strides ? out_strides[d] : run;
        run *= oshape[d] > 0 ? oshape[d] : 1;
    }
    j.shape[4] = 1;
    j.in = x;
    j.cosv = cosv;
    j.sinv = sinv;
    j.out = out;
    return j;
}

bool Instance::run_fused(const FusedGroup& fg) {
    const NodeDef& root = g.nodes[fg.root];
    Ctx c{*this, root};
    auto val = [&](int id) -> Tensor* {
        if (id < 0) return nullptr;
        Tensor& t = values[id];
        return t.present ? &t : nullptr;
    };
    rmlk_stream_t st = reinterpret_cast<rmlk_stream_t>(stream);
    switch (fg.kind) {
        case FusedGroup::RMSNORM: {
            Tensor *x = val(fg.v[0]), *w = val(fg.v[1]), *eps = val(fg.v[2]), *ex = val(fg.v[3]);
            Tensor *ra = val(fg.v[4]), *rb = val(fg.v[5]);  // the residual Add in front of the chain, if it joined
            const bool with_add = fg.v[4] >= 0;
            float e = 0.f, p = 0.f;
            if (with_add) {
                if (!ra || !rb || ra->dtype != RMLK_F32 || rb->dtype != RMLK_F32 || ra->shape != rb->shape || ra->parts > 1) return false;
                x = ra;  // same dtype and shape as the sum
            }
            if (!x || !w || !eps || !ex || x->dtype != RMLK_F32 || w->dtype != RMLK_F32 || x->shape.empty() || w->lazy) return false;
            if (!scalar_f32(*eps, e) || !scalar_f32(*ex, p)) return false;
            const int64_t cols = x->shape.back();
            if (cols == 0 || w->numel() != cols || w->shape.empty() || w->shape.back() != cols || w->shape.size() > x->shape.size()) return false;
            if (x->lazy) materialize(*x);
            const Shape oshape = x->shape;
            const int64_t rows = x->numel() / cols;
            if (!with_add) {
                Tensor& o = c.make(0, RMLK_F32, oshape);
                check_rc(rmlk_b200_rmsnorm(st, RMLK_F32, rows, cols, x->data, p, e, w->data, o.data));
                launches++;
                return true;
            }
            if (rb->lazy) materialize(*rb);
            Tensor& sum = values[fg.v[0]];
            sum.dtype = RMLK_F32;
            sum.shape = oshape;
            sum.mirror_valid = false;
            sum.mi.clear();
            sum.mf.clear();
            sum.lazy = false;
            sum.parts = 0;
            alloc_output(fg.v[0], sum);
            sum.present = true;
            Tensor& o = c.make(0, RMLK_F32, oshape);
            const int parts = rb->parts > 1 ? rb->parts : 1;
            check_rc(rmlk_b200_add_rmsnorm(st, RMLK_F32, rows, cols, ra->data, rb->data, parts, rows * cols, p, e, w->data, sum.data, o.data));
            launches++;
            if (rb->parts > 1) {  // the slabs have been consumed
                rb->parts = 0;
                rb->data = nullptr;
                rb->present = false;
                if (parts_owner == fg.v[5]) parts_owner = -1;
            }
            return true;
        }
        case FusedGroup::SWIGLU: {
            Tensor *gt = val(fg.v[0]), *up = val(fg.v[1]);
            if (!gt || !up || gt->dtype != RMLK_F32 || up->dtype != RMLK_F32 || gt->shape != up->shape) return false;
            // a view that is a block of columns of a wider matrix (one MatMul against concatenated weights) is read in place
            auto as_rows = [&](const Tensor& t, int64_t& pitch) {
                if (t.shape.empty()) return false;
                const int64_t cols = t.shape.back();
                if (!t.lazy) {
                    pitch = cols;
                    return true;
                }
                if (t.pshape.size() == 2 && t.pshape[1] == cols && t.pstride[1] == 1 && t.pshape[0] * cols == t.numel()) {
                    pitch = t.pstride[0];
                    return true;
                }
                if (t.pshape.size() == 1 && t.pshape[0] == cols && t.pstride[0] == 1 && t.numel() == cols) {
                    pitch = cols;
                    return true;
                }
                return false;
            };
            int64_t pg = 0, pu = 0;
            const bool pitched = (gt->lazy || up->lazy) && !gt->shape.empty() && gt->shape.back() % 4 == 0 && as_rows(*gt, pg) && as_rows(*up, pu) &&
                                 pg % 4 == 0 && pu % 4 == 0 && reinterpret_cast<uintptr_t>(gt->data) % 16 == 0 && reinterpret_cast<uintptr_t>(up->data) % 16 == 0;
            if (!pitched) {
                if (gt->lazy) materialize(*gt);
                if (up->lazy) materialize(*up);
            }
            const Shape oshape = gt->shape;
            const void *gd = gt->data, *ud = up->data;
            Tensor& o = c.make(0, RMLK_F32, oshape);
            if (o.numel() == 0) return true;
            if (pitched) {
                const int64_t cols = oshape.back();
                check_rc(rmlk_b200_swiglu_pitched(st, RMLK_F32, o.numel() / cols, cols, gd, pg, ud, pu, o.data));
            } else {
                check_rc(rmlk_b200_swiglu(st, RMLK_F32, o.numel(), gd, ud, o.data));
            }
            launches++;
            return true;
        }
        case FusedGroup::SCALE_MASK_SOFTMAX: {
            Tensor *s = val(fg.v[0]), *sc = val(fg.v[1]), *mk = val(fg.v[2]);
            float scale = 0.f;
            if (!s || !sc || !mk || s->dtype != RMLK_F32 || mk->dtype != RMLK_F32 || !scalar_f32(*sc, scale)) return false;
            const size_t rank = s->shape.size();
            if (rank < 1 || rank > 4 || mk->shape.size() > rank || mk->shape.empty()) return false;
            const int64_t axis = c.attr_int("axis", -1);
            if (axis != -1 && axis != static_cast<int64_t>(rank) - 1) return false;
            const int64_t cols = s->shape.back();
            if (cols == 0 || cols > 2048 || mk->shape.back() != cols) return false;
            if (mk->lazy) materialize(*mk);
            int64_t ms[4];
            if (!bcast_strides(*mk, s->shape, ms) || ms[rank - 1] != 1) return false;
            int64_t lead3[3] = {1, 1, 1}, mstr3[3] = {0, 0, 0};
            for (size_t d = 0; d + 1 < rank; d++) {
                lead3[3 - (rank - 1) + d] = s->shape[d];
                mstr3[3 - (rank - 1) + d] = ms[d];
            }
            if (s->lazy) materialize(*s);
            const Shape oshape = s->shape;
            Tensor& o = c.make(0, RMLK_F32, oshape);
            if (o.numel() == 0) return true;
            check_rc(rmlk_b200_scale_mask_softmax(st, RMLK_F32, lead3, cols, mstr3, scale, s->data, mk->data, o.data));
            launches++;
            return true;
        }
        case FusedGroup::ATTENTION: {
            Tensor *q = val(fg.v[0]), *sc = val(fg.v[1]), *mk = val(fg.v[2]), *kt = val(fg.v[3]), *vh = val(fg.v[4]);
            float scale = 0.f;
            if (!q || !sc || !mk || !kt || !vh || q->dtype != RMLK_F32 || mk->dtype != RMLK_F32 || kt->dtype != RMLK_F32 || vh->dtype != RMLK_F32 ||
                !scalar_f32(*sc, scale))
                return false;
            if (q->shape.size() != 4 || kt->shape.size() != 4 || vh->shape.size() != 4 || q->parts > 1) return false;
            const int64_t B = q->shape[0], H = q->shape[1], S = q->shape[2], D = q->shape[3], T = kt->shape[3];
            if (S != 1 || B <= 0 || H <= 0 || kt->shape[0] != B || kt->shape[1] != H || kt->shape[2] != D || vh->shape != Shape({B, H, T, D})) return false;
            {
                const NodeDef& smn = g.nodes[groups[fg.sub].root];
                const int64_t axis = Ctx{*this, smn}.attr_int("axis", -1);
                if (axis != -1 && axis != 3) return false;
            }
            // K^T and V must be views that repeat a dense [T, D] block per KV head over `fold` query heads
            LazyB lk, lv;
            if (!analyze_lazy_b(*kt, D, T, lk) || !lk.transposed || !analyze_lazy_b(*vh, T, D, lv) || lv.transposed) return false;
            if (lk.fold != lv.fold || lk.outer != lv.outer || lk.outer * lk.fold != B * H || H % lk.fold) return false;
            if (!rmlk_b200_gqa_decode_attention_supported(lk.fold, D, T)) return false;
            if (lk.outer > 1 && (lk.sb % 4 || lv.sb % 4)) return false;
            if (reinterpret_cast<uintptr_t>(kt->data) % 16 || reinterpret_cast<uintptr_t>(vh->data) % 16) return false;
            if (mk->lazy) materialize(*mk);
            int64_t ms[4];
            const Shape sshape = {B, H, 1, T};
            if (mk->shape.size() > 4 || mk->shape.empty() || mk->shape.back() != T || !bcast_strides(*mk, sshape, ms) || (T > 1 && ms[3] != 1)) return false;
            if (q->lazy) materialize(*q);
            const void *kdata = kt->data, *vdata = vh->data;
            Tensor& o = c.make(0, RMLK_F32, Shape({B, H, 1, D}));
            // one CTA per problem in one pass over K and V by default; RMLK_B200_ATTENTION=split: keys split over CTAs, merged through a workspace
            const size_t ws_need = attention_split ? rmlk_b200_gqa_decode_attention_workspace_bytes(lk.outer, lk.fold, D, T) : 0;
            void* ws = nullptr;
            if (ws_need) {
                ws = attn_ws.ensure(ws_need);
                // The arrival counters (16 bytes per problem at the start of the workspace) must be zero when the kernel
                // starts; the kernel leaves them at zero.  A new buffer is cleared whole.  When the number of problems
                // changes the layout moves - last run's partial sums may lie where this run's counters are - so the
                // counter prefix is cleared again.
                const size_t counter_bytes = static_cast<size_t>(lk.outer) * 16;
                if (attn_ws.cap != attn_ws_zeroed) {
                    check_cuda(cudaMemsetAsync(attn_ws.ptr, 0, attn_ws.cap, stream), "attention workspace clear");
                    attn_ws_zeroed = attn_ws.cap;
                } else if (lk.outer != attn_ws_problems) {
                    check_cuda(cudaMemsetAsync(attn_ws.ptr, 0, counter_bytes < attn_ws.cap ? counter_bytes : attn_ws.cap, stream), "attention counters clear");
                }
                attn_ws_problems = lk.outer;
            }
            check_rc(rmlk_b200_gqa_decode_attention_ws(st, RMLK_F32, lk.outer, lk.fold, D, T, H / lk.fold, q->data, kdata, lk.sb, vdata, lv.sb, scale,
                                                       mk->data, ms[0], ms[1], o.data, ws, ws_need));
            launches++;
            return true;
        }
        case FusedGroup::MASK: {
            Tensor *am = val(fg.v[0]), *shp = val(fg.v[1]);
            Tensor* kt = fg.v[2] >= 0 ? val(fg.v[2]) : nullptr;
            if (!am || !shp || am->dtype != RMLK_I64 || am->shape.size() != 2 || shp->dtype != RMLK_I64) return false;
            if (fg.v[2] >= 0 && (!kt || !kt->is_scalar() || kt->dtype != RMLK_I64)) return false;
            float c1, yv, zv, c0, xv;
            Tensor *t3 = val(fg.v[3]), *t4 = val(fg.v[4]), *t5 = val(fg.v[5]), *t6 = val(fg.v[6]), *t7 = val(fg.v[7]);
            if (!t3 || !t4 || !t5 || !t6 || !t7 || !scalar_f32(*t3, c1) || !scalar_f32(*t4, yv) || !scalar_f32(*t5, zv) || !scalar_f32(*t6, c0) ||
                !scalar_f32(*t7, xv))
                return false;
            // the chain's own attributes: f32 fill value, upper triangle, Cast to f32, Unsqueeze axes [0, 1] and [1, 2]
            float fill = 0.0f;
            {
                const Ctx cc{*this, g.nodes[fg.v[8]]};
                if (const Attr* a = cc.attr("value")) {
                    if (a->kind != Attr::TENSOR || a->t_dtype != RMLK_F32 || a->t_data.size() < 4) return false;
                    std::memcpy(&fill, a->t_data.data(), 4);
                }
                if (Ctx{*this, g.nodes[fg.v[9]]}.attr_int("upper", 1) == 0) return false;
            }
            for (int mnode : fg.members)
                if (g.nodes[mnode].op == RMLK_OP_CAST) {
                    const Attr* to = Ctx{*this, g.nodes[mnode]}.attr("to");
                    if (!to || to->kind != Attr::INT || onnx_to_dtype(to->i) != RMLK_F32) return false;
                }
            auto axes_are = [&](int node, int64_t a0, int64_t a1) {
                const Ctx cu{*this, g.nodes[node]};
                std::vector<int64_t> axes;
                if (Tensor* at = cu.in(1)) axes = host_i64(*at);
                else if (const Attr* a = cu.attr("axes")) axes = a->ints;
                return axes.size() == 2 && axes[0] == a0 && axes[1] == a1;
            };
            if (!axes_are(fg.v[10], 0, 1) || !axes_are(fg.v[11], 1, 2)) return false;
            const std::vector<int64_t> dims = host_i64(*shp);
            if (dims.size() != 2 || dims[0] < 0 || dims[1] < 0 || dims[1] != am->shape[1]) return false;
            const int64_t k = kt ? host_i64(*kt)[0] : 0;
            if (am->lazy) materialize(*am);
            const int64_t B = am->shape[0], S = dims[0], T = dims[1];
            const void* amd = am->data;
            Tensor& o = c.make(0, RMLK_F32, Shape{B, 1, S, T});
            if (o.numel() == 0) return true;
            check_rc(rmlk_b200_causal_padding_mask(st, B, S, T, k, amd, fill, c1, yv, zv, c0, xv, o.data));
            launches++;
            return true;
        }
        case FusedGroup::ROPE_TABLES: {
            Tensor *p0 = val(fg.v[0]), *p1 = val(fg.v[1]);
            if (!p0 || !p1 || p0->dtype != RMLK_F32 || p1->dtype != RMLK_F32) return false;
            // one operand holds one value per row ([..., 1]), the other one value per column ([half]); either order
            Tensor *a = p0, *b = p1;
            if (!(a->shape.size() >= 1 && a->shape.back() == 1)) std::swap(a, b);
            if (a->shape.empty() || a->shape.back() != 1 || b->shape.size() != 1 || b->numel() < 1) return false;
            if (a->lazy) {
                // a regrouped view of a dense tensor (Unsqueeze) reads like the dense tensor; anything else is copied out
                Shape ps, pst;
                std::vector<std::pair<int, int>> gr;
                bool dense = dims_of(*a, ps, pst, gr);
                int64_t run = 1;
                for (int d = static_cast<int>(ps.size()) - 1; d >= 0 && dense; d--) {
                    if (ps[d] != 1 && pst[d] != run) dense = false;
                    run *= ps[d];
                }
                if (!dense) materialize(*a);
            }
            if (b->lazy) materialize(*b);
            const int64_t rows = a->numel(), half = b->numel();
            Shape oshape = a->shape;
            oshape.back() = 2 * half;
            const void *ad = a->data, *bd = b->data;
            Tensor& oc = Ctx{*this, g.nodes[fg.v[2]]}.make(0, RMLK_F32, oshape);
            Tensor& os = Ctx{*this, g.nodes[fg.v[3]]}.make(0, RMLK_F32, oshape);
            if (rows == 0) return true;
            check_rc(rmlk_b200_rope_tables(st, RMLK_F32, rows, half, ad, bd, oc.data, os.data));
            launches++;
            return true;
        }
        case FusedGroup::ROPE: {
            Tensor *x = val(fg.v[0]), *cs = val(fg.v[1]), *sn = val(fg.v[2]);
            if (!x || !cs || !sn || x->dtype != RMLK_F32 || cs->dtype != RMLK_F32 || sn->dtype != RMLK_F32 || x->shape.size() != 4) return false;
            const int64_t D = x->shape[3];
            if (D < 2 || D % 2) return false;
            // the two Slice nodes must cut [0, D/2) and [D/2, D) of the last axis with step 1; the Concat joins on it
            auto slice_ok = [&](int node, int64_t lo, int64_t hi) {
                const NodeDef& n = g.nodes[node];
                Tensor *s0 = val(n.inputs[1]), *e0 = val(n.inputs[2]), *a0 = val(n.inputs[3]);
                Tensor* p0 = n.inputs.size() > 4 ? val(n.inputs[4]) : nullptr;
                if (!s0 || !e0 || !a0 || !small_mirrored(*s0) || !small_mirrored(*e0) || !small_mirrored(*a0)) return false;
                if (s0->mi.size() != 1 || e0->mi.size() != 1 || a0->mi.size() != 1) return false;
                if (p0 && (!small_mirrored(*p0) || p0->mi.size() != 1 || p0->mi[0] != 1)) return false;
                if (n.inputs.size() > 4 && n.inputs[4] >= 0 && !p0) return false;
                const int64_t ax = a0->mi[0];
                return (ax == 3 || ax == -1) && s0->mi[0] == lo && (e0->mi[0] == hi || (hi == D && e0->mi[0] >= D));
            };
            if (!slice_ok(fg.v[3], 0, D / 2) || !slice_ok(fg.v[4], D / 2, D)) return false;
            const int64_t cat_axis = Ctx{*this, g.nodes[fg.v[5]]}.attr_int("axis", 0);
            if (cat_axis != 3 && cat_axis != -1) return false;
            if (cs->lazy) materialize(*cs);
            if (sn->lazy) materialize(*sn);
            int64_t cstr[4], sstr[4], xstr[4];
            if (!bcast_strides(*cs, x->shape, cstr) || !bcast_strides(*sn, x->shape, sstr)) return false;
            // x may be a permuted view: one physical dim (or none) per logical dim, else copy it out first
            bool strided_ok = false;
            if (x->lazy) {
                std::vector<std::pair<int, int>> groups_;
                Shape xps, xpst;
                if (dims_of(*x, xps, xpst, groups_)) {
                    strided_ok = true;
                    for (int d = 0; d < 4 && strided_ok; d++) {
                        int cnt = 0;
                        xstr[d] = 0;
                        for (int p = groups_[d].first; p < groups_[d].second; p++)
                            if (xps[p] != 1) {
                                cnt++;
                                xstr[d] = xpst[p];
                            }
                        strided_ok = cnt <= 1;
                    }
                }
                if (!strided_ok) materialize(*x);
            }
            if (!strided_ok) {
                const Shape st4 = dense_strides(x->shape);
                for (int d = 0; d < 4; d++) xstr[d] = st4[d];
            }
            const Shape oshape = x->shape;
            const void* xdata = x->data;
            // rotated keys that are only ever appended to a carried cache are written straight into their slot
            const int ov = root.outputs[0];
            const int cnode = ov < static_cast<int>(append_consumer.size()) ? append_consumer[ov] : -1;
            void* slot = nullptr;
            Shape ost;
            if (cnode >= 0 && x->numel() > 0 && append_slot_for(*this, cnode, RMLK_F32, oshape, slot, ost)) {
                Tensor& o = c.out(0);
                o.dtype = RMLK_F32;
                o.shape = oshape;
                o.mirror_valid = false;
                o.mi.clear();
                o.mf.clear();
                o.parts = 0;
                set_strided(o, slot, oshape, ost);
                o.present = true;
                defer_job(rope_job(oshape, xstr, cstr, sstr, xdata, cs->data, sn->data, slot, ost.data()));
                return true;
            }
            Tensor& o = c.make(0, RMLK_F32, oshape);
            if (o.numel() == 0) return true;
            defer_job(rope_job(oshape, xstr, cstr, sstr, xdata, cs->data, sn->data, o.data, nullptr));
            return true;
        }
    }
    return false;
}

// ---------------------------------------------------------------------------------------------
// MatMul nodes sharing their left operand, against constant weights: one MatMul on concatenated weights
// ---------------------------------------------------------------------------------------------
void Instance::find_merged_matmuls() {
    merged.clear();
    merged_of_node.assign(g.nodes.size(), -1);
    if (getenv("RMLK_B200_NO_MATMUL_MERGE")) return;
    std::map<std::pair<int, int64_t>, std::vector<int>> by_input;  // (left operand, K) -> nodes
    for (size_t i = 0; i < g.nodes.size(); i++) {
        const NodeDef& n = g.nodes[i];
        if (n.op != RMLK_OP_MATMUL || n.inputs.size() < 2 || n.outputs.empty() || n.inputs[0] < 0 || n.inputs[1] < 0) continue;
        const ValueDef& w = g.values[n.inputs[1]];
        const ValueDef& o = g.values[n.outputs[0]];
        if (!w.is_const || w.dtype != RMLK_F32 || w.dims.size() != 2 || w.dims[0] <= 0 || w.dims[1] <= 0 || w.dims[1] % 4) continue;
        if (o.is_output || g.values[n.inputs[0]].is_const) continue;
        by_input[{n.inputs[0], w.dims[0]}].push_back(static_cast<int>(i));
    }
    for (auto& kv : by_input) {
        if (kv.second.size() < 2) continue;
        MergedMatMul mm;
        mm.nodes = kv.second;
        mm.a_value = kv.first.first;
        mm.k = kv.first.second;
        for (int node : mm.nodes) {
            const int64_t n = g.values[g.nodes[node].inputs[1]].dims[1];
            mm.col0.push_back(mm.n_total);
            mm.n.push_back(n);
            mm.n_total += n;
        }
        for (int node : mm.nodes) merged_of_node[node] = static_cast<int>(merged.size());
        merged.push_back(std::move(mm));
    }
}

// Called for a member node.  True: the node's output is in place (produced now, or earlier in this run by the
// group's first member).  False: the tensors of this run do not fit; the node runs as an ordinary MatMul.
bool Instance::run_merged_matmul(int node_index) {
    MergedMatMul& mm = merged[merged_of_node[node_index]];
    if (mm.done_in_run == run_counter) return node_index != mm.nodes.front() ? values[g.nodes[node_index].outputs[0]].present : false;
    if (node_index != mm.nodes.front()) return false;  // the first member decided against it for this run
    Tensor& a = values[mm.a_value];
    if (!a.present || a.dtype != RMLK_F32 || a.shape.empty() || a.shape.back() != mm.k || a.numel() == 0) return false;
    for (size_t j = 0; j < mm.nodes.size(); j++) {
        const Tensor& w = values[g.nodes[mm.nodes[j]].inputs[1]];
        if (!w.present || w.lazy || w.dtype != RMLK_F32 || w.shape.size() != 2 || w.shape[0] != mm.k || w.shape[1] != mm.n[j]) return false;
    }
    if (a.lazy) materialize(a);
    const int flags = mm.ready ? RMLK_MATMUL_B_STATIC : 0;  // from the second run on nothing in flight writes the weights
    if (!mm.ready) {
        char* dst = static_cast<char*>(mm.w.ensure(static_cast<size_t>(mm.k) * mm.n_total * sizeof(float)));
        for (size_t j = 0; j < mm.nodes.size(); j++) {
            const Tensor& w = values[g.nodes[mm.nodes[j]].inputs[1]];
            check_cuda(cudaMemcpy2DAsync(dst + mm.col0[j] * sizeof(float), mm.n_total * sizeof(float), w.data, mm.n[j] * sizeof(float),
                                         mm.n[j] * sizeof(float), static_cast<size_t>(mm.k), cudaMemcpyDeviceToDevice, stream), "weight concatenation");
        }
        mm.ready = true;
    }
    const int64_t rows = a.numel() / mm.k;
    Storage* y = arena->alloc(static_cast<size_t>(rows) * mm.n_total * sizeof(float));
    const size_t need = rmlk_b200_matmul_workspace_bytes(RMLK_F32, 1, rows, mm.n_total, mm.k);
    void* ws = need ? matmul_ws.ensure(need) : nullptr;
    if (batch_jobs && rows <= 64) {
        // decode-sized product: the split-K slabs stay unsummed for the placements that read them (Instance::unsummed)
        int parts = 1;
        check_rc(rmlk_b200_matmul_parts(reinterpret_cast<rmlk_stream_t>(stream), RMLK_F32, rows, mm.n_total, mm.k, a.data, mm.w.ptr, y->ptr, ws, need,
                                        static_cast<int*>(status_word.ptr), flags, &parts));
        launches++;
        if (parts > 1) {
            unsummed.y = y;
            unsummed.slabs = static_cast<const float*>(ws);
            unsummed.parts = parts;
            unsummed.part_stride = rows * mm.n_total;
            y->refs++;
        }
    } else {
        check_rc(rmlk_b200_matmul_flags(reinterpret_cast<rmlk_stream_t>(stream), RMLK_F32, 1, rows, mm.n_total, mm.k, a.data, 0, mm.w.ptr, 0, y->ptr,
                                        rows * mm.n_total, ws, need, static_cast<int*>(status_word.ptr), flags));
        launches += need ? 2 : 1;
    }
    status_dirty = true;
    for (size_t j = 0; j < mm.nodes.size(); j++) {
        Tensor& o = values[g.nodes[mm.nodes[j]].outputs[0]];
        o.dtype = RMLK_F32;
        o.shape.assign(a.shape.begin(), a.shape.end() - 1);  // [..., M, K] x [K, N_j] -> [..., M, N_j]
        o.shape.push_back(mm.n[j]);
        o.mirror_valid = false;
        o.mi.clear();
        o.mf.clear();
        o.data = static_cast<char*>(y->ptr) + mm.col0[j] * sizeof(float);
        o.storage = y;
        if (j > 0) y->refs++;
        o.pshape.clear();
        o.pstride.clear();
        o.lazy = rows > 1;
        if (o.lazy) {
            push_dim(o.pshape, o.pstride, rows, mm.n_total);
            push_dim(o.pshape, o.pstride, mm.n[j], 1);
        }
        o.present = true;
    }
    mm.done_in_run = run_counter;
    return true;
}

void Instance::run_node(const NodeDef& n) {
    if (!merged_of_node.empty()) {
        const int idx = static_cast<int>(&n - g.nodes.data());
        if (idx >= 0 && idx < static_cast<int>(g.nodes.size()) && merged_of_node[idx] >= 0 && run_merged_matmul(idx)) return;
    }
    Ctx c{*this, n};
    switch (n.op) {
        case RMLK_OP_NOOP: case RMLK_OP_CONST: return;
        case RMLK_OP_ADD: return op_binary(c, RMLK_BIN_ADD);
        case RMLK_OP_SUB: return op_binary(c, RMLK_BIN_SUB);
        case RMLK_OP_MUL: return op_binary(c, RMLK_BIN_MUL);
        case RMLK_OP_DIV: return op_binary(c, RMLK_BIN_DIV);
        case RMLK_OP_EQUAL: return op_binary(c, RMLK_BIN_EQUAL);
        case RMLK_OP_GREATER: return op_binary(c, RMLK_BIN_GREATER);
        case RMLK_OP_POW: return op_pow(c);
        case RMLK_OP_SQRT: return op_unary(c, RMLK_UN_SQRT);
        case RMLK_OP_NEG: return op_unary(c, RMLK_UN_NEG);
        case RMLK_OP_SIN: return op_unary(c, RMLK_UN_SIN);
        case RMLK_OP_COS: return op_unary(c, RMLK_UN_COS);
        case RMLK_OP_SIGMOID: return op_unary(c, RMLK_UN_SIGMOID);
        case RMLK_OP_RELU: return op_unary(c, RMLK_UN_RELU);
        case RMLK_OP_CAST: return op_cast(c);
        case RMLK_OP_WHERE: return op_where(c);
        case RMLK_OP_REDUCE_MEAN: return op_reduce_mean(c);
        case RMLK_OP_SOFTMAX: return op_softmax(c);
        case RMLK_OP_MATMUL: return op_matmul(c);
        case RMLK_OP_GEMM: return op_gemm(c);
        case RMLK_OP_GATHER: return op_gather(c);
        case RMLK_OP_SCATTER_ND: return op_scatter_nd(c);
        case RMLK_OP_SLICE: return op_slice(c);
        case RMLK_OP_TRANSPOSE: return op_transpose(c);
        case RMLK_OP_CONCAT: return op_concat(c);
        case RMLK_OP_EXPAND: return op_expand(c);
        case RMLK_OP_TRILU: return op_trilu(c);
        case RMLK_OP_RANGE: return op_range(c);
        case RMLK_OP_RESHAPE: return op_reshape(c);
        case RMLK_OP_UNSQUEEZE: return op_unsqueeze(c);
        case RMLK_OP_FLATTEN: return op_flatten(c);
        case RMLK_OP_SHAPE: return op_shape(c);
        case RMLK_OP_CONSTANT_OF_SHAPE: return op_constant_of_shape(c);
        case RMLK_OP_CONSTANT: return;  // materialised at instance creation
        default:
            raise(RMLK_ERR_INVALID_ARG, "op " + std::to_string(n.op) + " is outside the operator path this library implements");
    }
}

}  // namespace rt
}  // namespace rmlk
