// Lazy Tensor mirror for the dense path.
//
// morok's `Tensor` records operations in a graph and computes on `realize()`
// (tensor/src/realize.rs:83-127: schedule -> allocate -> prepare kernels -> ExecutionPlan::execute,
// runtime/src/execution_plan.rs:168-181).  The reference lowers that graph to generated code; this
// mirror lowers it to calls of the library's kernels:
//   * nodes are created by the mk_tensor_* constructors and hold shared pointers to their inputs;
//   * realize() walks the graph in post-order, takes output buffers from the LRU allocator, and
//     issues one kernel call per node on the device's default stream, in topological order;
//   * movement ops (reshape / permute) are views: strides change, no kernel runs.  A consumer that
//     cannot read strides (GEMM needs rows with unit inner stride; element-wise ops need dense
//     data) makes one gathering copy; attention reads [B,S,H,D]-stored operands in place;
//   * the same local fusions the reference gets from keeping an expression in one kernel are
//     applied at realize time: add(x, matmul(a, b)) -> GEMM with the add in its epilogue
//     (tensor/src/test/unit/fusion.rs:21-27; x may also be `linear`'s bias of N elements), mul(silu(g), u) -> one SwiGLU kernel
//     (fusion.rs:58-67, 106-114; when g and u are matmuls of the same input, the gate moves into the store of one
//     GEMM kernel that computes both), permute(0,2,1,3) of an attention output -> attention stores in that
//     layout directly, cast(rms_norm(x)) back to x's 16-bit type -> one norm kernel;
//   * once a node is realized it drops its inputs, so intermediates return to the allocator
//     cache as soon as nothing else refers to them (tensor/src/realize.rs:199-233).
// Binary ops promote mixed dtypes to f32 like least_upper_dtype does for (bf16|f16, f32)
// (dtype/src/cast.rs:5-20): rms_norm of a bf16 tensor therefore yields f32, as in the reference
// (tensor/src/nn/norm.rs:92-110).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>

#include "mk_internal.h"

using namespace mk;

namespace {

enum Op { LEAF, MATMUL, SDPA, RMSNORM, ROPE, SILU, SIGMOID, ADD, MUL, CAST, VIEW };

struct Node {
    Op op = LEAF;
    mk_device* dev = nullptr;
    int32_t dtype = MK_F32;
    std::vector<int64_t> shape;
    std::vector<std::shared_ptr<Node>> in;
    // attributes
    float eps = 0, scale = 0, softcap = 0;
    int causal = 0, interleaved = 0;
    int64_t row_div = 1;               // ROPE: input rows that share one cos/sin table row
    // storage (set once realized; views share the producer's allocation)
    bool realized = false;
    std::shared_ptr<mk_buf> buf;       // owning handle (freed -> allocator cache)
    std::vector<int64_t> strides;      // element strides; valid once realized
    int64_t offset = 0;                // element offset into buf
    // VIEW: how this node's index space maps onto its input (resolved at realize time)
    std::vector<int64_t> view_shape;   // == shape
    std::vector<int32_t> perm;         // non-empty: permute of input axes; empty: reshape
    int32_t last_launches = 0;
    // Set while a plan was being recorded: the node has a buffer but no data until the plan has run once
    // (the flag is the plan's "has run" marker, shared by every node the recording realized).
    std::shared_ptr<std::atomic<bool>> plan_ran;
    bool has_data() const { return realized && (!plan_ran || plan_ran->load()); }

    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    int ndim() const { return (int)shape.size(); }
};

using NodeP = std::shared_ptr<Node>;

std::vector<int64_t> contiguous_strides(const std::vector<int64_t>& shape) {
    std::vector<int64_t> s(shape.size());
    int64_t acc = 1;
    for (int i = (int)shape.size() - 1; i >= 0; --i) {
        s[i] = acc;
        acc *= shape[i];
    }
    return s;
}

bool is_contiguous(const Node& n) {
    int64_t acc = 1;
    for (int i = n.ndim() - 1; i >= 0; --i) {
        if (n.shape[i] != 1 && n.strides[i] != acc) return false;
        acc *= n.shape[i];
    }
    return true;
}

// realize() issues its kernels on this stream: the default stream normally, the capturing stream while
// mk_tensor_compile records a plan.  While a plan is recorded, every buffer realize() takes is also kept
// in t_retain: the plan's kernels have those addresses baked in, so the buffers must neither return to
// the allocator cache nor be handed to anyone else for as long as the plan lives.
thread_local mk_stream* t_stream = nullptr;
thread_local std::vector<std::shared_ptr<mk_buf>>* t_retain = nullptr;
thread_local std::shared_ptr<std::atomic<bool>> t_plan_ran;      // the recording plan's marker (null outside recording)

std::shared_ptr<mk_buf> make_buf(mk_device* dev, size_t bytes, mk_status* st) {
    mk_buf* b = nullptr;
    *st = mk_alloc(dev, bytes, 0, &b);
    if (*st != MK_OK) return nullptr;
    std::shared_ptr<mk_buf> sp(b, [](mk_buf* x) { mk_free(x); });
    if (t_retain) t_retain->push_back(sp);
    return sp;
}

mk_status node_ptr(const Node& n, void** out) {
    void* base = nullptr;
    mk_status st = n.numel() == 0 ? MK_OK : buf_ptr(n.buf.get(), &base);
    if (st != MK_OK) return st;
    // a recording plan bakes this address into its kernels: keep the buffer (leaf inputs included) alive with the plan
    if (t_retain && n.buf && (t_retain->empty() || t_retain->back() != n.buf)) t_retain->push_back(n.buf);
    *out = base ? (char*)base + n.offset * (int64_t)dtype_size(n.dtype) : nullptr;
    return MK_OK;
}

mk_status alloc_output(Node& n) {
    mk_status st;
    n.buf = make_buf(n.dev, (size_t)n.numel() * dtype_size(n.dtype), &st);
    if (st != MK_OK) return st;
    n.strides = contiguous_strides(n.shape);
    n.offset = 0;
    return MK_OK;
}

mk_status realize(const NodeP& n);

// Returns a node with the same values as `n` whose data is dense row-major (gathers if needed).
mk_status dense(const NodeP& n, NodeP* out) {
    mk_status st = realize(n);
    if (st != MK_OK) return st;
    if (is_contiguous(*n)) {
        *out = n;
        return MK_OK;
    }
    auto c = std::make_shared<Node>();
    c->op = LEAF;
    c->dev = n->dev;
    c->dtype = n->dtype;
    c->shape = n->shape;
    st = alloc_output(*c);
    if (st != MK_OK) return st;
    void *src, *dst;
    if ((st = node_ptr(*n, &src)) != MK_OK || (st = node_ptr(*c, &dst)) != MK_OK) return st;
    MK_REQUIRE(n->ndim() <= MK_MAX_DIMS, "tensor: more than %d dimensions", MK_MAX_DIMS);
    st = strided_copy(n->dev, raw(t_stream), (int)dtype_size(n->dtype), src, dst, n->ndim(), n->shape.data(), n->strides.data());
    if (st != MK_OK) return st;
    c->realized = true;
    c->plan_ran = t_plan_ran;
    *out = c;
    return MK_OK;
}

// ---- per-op lowering ---------------------------------------------------------------------------------
// The gated pair act(a b + bias_gate) * (a b2 + bias_up) of two products over the same input.
struct GateSpec {
    NodeP b2;                    // weights of the second product
    NodeP bias_gate, bias_up;    // null or N elements each
    bool sigmoid = false;        // act = sigmoid instead of silu
};

// gate set: the gated pair in one kernel; `*fell_back` reports that the shapes or the device did not allow
// it (nothing has been launched then and n has no buffer).
mk_status run_matmul(Node& n, const NodeP& a_in, const NodeP& b_in, const NodeP& addend, const GateSpec* gate = nullptr, bool* fell_back = nullptr) {
    // Shapes follow tensor/src/matmul.rs:82-110: a [..., M, K] (or [K]), b [..., K, N] (or [K]).
    NodeP a, b = b_in;
    mk_status st = dense(a_in, &a);
    if (st != MK_OK) return st;
    st = realize(b);
    if (st != MK_OK) return st;
    const int64_t K = a->shape.back();
    const bool b_vec = b->ndim() == 1;
    const int64_t N = b_vec ? 1 : b->shape.back();
    // `linear` hands over weights as a transposed view of [N, K] storage: run it as trans_b.
    int trans_b = 0;
    int64_t ldb = 0;
    if (b->ndim() == 2 && b->strides[1] == 1 && b->strides[0] >= N) {
        ldb = b->strides[0];
    } else if (b->ndim() == 2 && b->strides[0] == 1 && b->strides[1] >= K && b->shape[1] > 1) {
        trans_b = 1;
        ldb = b->strides[1];
    } else {
        NodeP bd;
        st = dense(b, &bd);
        if (st != MK_OK) return st;
        b = bd;
        ldb = N;
    }
    int64_t M, batch = 1, stride_a = 0, stride_b = 0;
    if (b->ndim() <= 2) {
        M = n.numel() / std::max<int64_t>(N, 1);   // a's leading dimensions flatten into rows
    } else {
        // batched: leading dims of b must equal a's (or a is 2-D and broadcasts)
        M = a->ndim() >= 2 ? a->shape[a->ndim() - 2] : 1;
        batch = 1;
        for (int i = 0; i < b->ndim() - 2; ++i) batch *= b->shape[i];
        stride_b = K * N;
        if (a->ndim() == b->ndim()) {
            for (int i = 0; i < a->ndim() - 2; ++i)
                if (a->shape[i] != b->shape[i]) return fail(MK_ERR_UNSUPPORTED, "matmul: batch dimensions must match (broadcast of size-1 batch dims is not supported)");
            stride_a = M * K;
        } else if (a->ndim() <= 2) {
            stride_a = 0;
        } else {
            return fail(MK_ERR_UNSUPPORTED, "matmul: unsupported batch broadcast");
        }
    }
    mk_gemm_desc d{};
    d.dtype_in = a->dtype;
    d.dtype_out = n.dtype;
    d.M = M; d.N = N; d.K = K;
    d.lda = K;
    d.ldb = ldb;
    d.ldc = N;
    d.trans_b = trans_b;
    d.batch = (int32_t)batch;
    d.stride_a = stride_a; d.stride_b = stride_b; d.stride_c = M * N;
    void *pa, *pb, *pc, *pd = nullptr;
    if ((st = node_ptr(*a, &pa)) != MK_OK || (st = node_ptr(*b, &pb)) != MK_OK) return st;
    NodeP add_dense;
    if (addend) {
        if ((st = dense(addend, &add_dense)) != MK_OK || (st = node_ptr(*add_dense, &pd)) != MK_OK) return st;
        // a full-size addend is a residual; one of N elements is a bias added to every row
        d.epilogue = (add_dense->numel() == n.numel()) ? MK_EPI_ADD : MK_EPI_ADD_ROW;
        d.D = pd;
    }
    NodeP bias_dense[2];
    if (gate) {
        // the second weight matrix must look exactly like the first (same orientation and leading dimension)
        NodeP b2 = gate->b2;
        if ((st = realize(b2)) != MK_OK) return st;
        const bool same = b2->ndim() == 2 && b->ndim() == 2 && b2->shape == b->shape && b2->strides == b->strides && b2->dtype == b->dtype && batch == 1;
        void* pb2 = nullptr;
        if (!same || (st = node_ptr(*b2, &pb2)) != MK_OK) {
            *fell_back = true;
            return MK_OK;
        }
        d.epilogue = MK_EPI_SWIGLU;
        d.B2 = pb2;
        if (gate->sigmoid) d.flags |= MK_GEMM_GATE_SIGMOID;
        const NodeP* biases[2] = {&gate->bias_gate, &gate->bias_up};
        for (int i = 0; i < 2; ++i) {
            if (!*biases[i]) continue;
            void* pbias = nullptr;
            if ((st = dense(*biases[i], &bias_dense[i])) != MK_OK || (st = node_ptr(*bias_dense[i], &pbias)) != MK_OK) return st;
            (i == 0 ? d.D : d.D2) = pbias;
        }
    }
    if ((st = alloc_output(n)) != MK_OK || (st = node_ptr(n, &pc)) != MK_OK) return st;
    d.A = pa; d.B = pb; d.C = pc;
    if (n.numel() == 0) return MK_OK;
    st = mk_gemm(n.dev, t_stream, &d);
    if (gate && st == MK_ERR_UNSUPPORTED) {   // not a tensor-core shape: the caller runs the three kernels instead
        n.buf.reset();
        *fell_back = true;
        return MK_OK;
    }
    return st;
}

// Strides (batch, head, row) of a 4-D [B,H,S,D] tensor whose last dimension is dense, else false.
bool bhsd_strides(const Node& t, int64_t out[3]) {
    if (t.ndim() != 4 || (t.shape[3] != 1 && t.strides[3] != 1)) return false;
    out[0] = t.strides[0]; out[1] = t.strides[1]; out[2] = t.strides[2];
    return true;
}

mk_status run_sdpa(Node& n, bool store_bshd) {
    NodeP q = n.in[0], k = n.in[1], v = n.in[2], mask = n.in.size() > 3 ? n.in[3] : nullptr;
    mk_status st;
    NodeP t[3] = {q, k, v};
    int64_t strides[3][3];
    for (int i = 0; i < 3; ++i) {
        if ((st = realize(t[i])) != MK_OK) return st;
        if (!bhsd_strides(*t[i], strides[i])) {
            NodeP dn;
            if ((st = dense(t[i], &dn)) != MK_OK) return st;
            t[i] = dn;
            bhsd_strides(*t[i], strides[i]);
        }
    }
    mk_sdpa_desc d{};
    d.dtype = n.dtype;
    d.B = (int32_t)q->shape[0]; d.Hq = (int32_t)q->shape[1]; d.Hkv = (int32_t)k->shape[1];
    d.Sq = (int32_t)q->shape[2]; d.Sk = (int32_t)k->shape[2]; d.D = (int32_t)q->shape[3]; d.Dv = (int32_t)v->shape[3];
    d.scale = n.scale; d.causal = n.causal; d.softcap = n.softcap;
    for (int i = 0; i < 3; ++i) { d.q_strides[i] = strides[0][i]; d.k_strides[i] = strides[1][i]; d.v_strides[i] = strides[2][i]; }
    void *pq, *pk, *pv, *po, *pm = nullptr;
    if ((st = node_ptr(*t[0], &pq)) != MK_OK || (st = node_ptr(*t[1], &pk)) != MK_OK || (st = node_ptr(*t[2], &pv)) != MK_OK) return st;
    NodeP md;
    if (mask) {
        if ((st = dense(mask, &md)) != MK_OK || (st = node_ptr(*md, &pm)) != MK_OK) return st;
        d.mask = pm;
        // the mask broadcasts against [B, H, Sq, Sk] (tensor/src/transformer.rs:112-124): right-align its shape, a
        // dimension of 1 repeats (stride 0), the others step through the dense data
        d.mask_kind = md->dtype == MK_BOOL ? MK_MASK_BOOL : MK_MASK_F32;
        const int lead = 4 - md->ndim();
        int64_t acc = md->shape.back();       // == Sk (checked when the graph was built)
        for (int dim = 2; dim >= 0; --dim) {  // query row, head, batch
            const int j = dim - lead;         // index into the mask's own shape
            const int64_t extent = j >= 0 ? md->shape[j] : 1;
            d.mask_strides[dim] = extent == 1 ? 0 : acc;
            acc *= extent;
        }
    }
    if ((st = alloc_output(n)) != MK_OK || (st = node_ptr(n, &po)) != MK_OK) return st;
    const int64_t H = d.Hq, S = d.Sq, Dv = d.Dv;
    if (store_bshd) {   // memory order [B,S,H,Dv]; the node itself stays indexed [B,H,S,Dv]
        n.strides = {S * H * Dv, Dv, H * Dv, 1};
    }
    d.o_strides[0] = n.strides[0]; d.o_strides[1] = n.strides[1]; d.o_strides[2] = n.strides[2];
    d.Q = pq; d.K = pk; d.V = pv; d.O = po;
    if (n.numel() == 0) return MK_OK;
    return mk_sdpa_fwd(n.dev, t_stream, &d);
}

mk_status run_binary(Node& n) {
    const bool mul = n.op == MUL;
    mk_status st;
    NodeP a = n.in[0], b = n.in[1];
    // fusions (see the header comment)
    if (!mul) {
        for (int side = 0; side < 2; ++side) {
            const NodeP& mm = n.in[side];
            const NodeP& other = n.in[1 - side];
            if (mm->op != MATMUL || mm->realized) continue;
            const bool residual = other->shape == n.shape;
            const bool bias = other->ndim() == 1 && other->shape[0] == n.shape.back() && mm->in[1]->ndim() == 2;   // `linear`'s bias
            if (mm->dtype == n.dtype && mm->shape == n.shape && other->dtype == n.dtype && (residual || bias))
                return run_matmul(n, mm->in[0], mm->in[1], other);
        }
    } else {
        // mul(act(x w1 [+ b1]), x w2 [+ b2]) over the same x, act = silu or sigmoid: one GEMM kernel that keeps both
        // products in tensor memory and applies biases and gate in its store
        // (tensor/src/test/unit/fusion.rs:58-67, 106-114); the operands may come in either order
        for (int side = 0; side < 2; ++side) {
            const NodeP& act = n.in[side];
            const NodeP& up = n.in[1 - side];
            if ((act->op != SILU && act->op != SIGMOID) || act->realized || act->shape != up->shape || n.dtype == MK_F32) continue;
            // a product, optionally plus a bias row of N elements (`linear` with a bias)
            auto product = [&](const NodeP& t, NodeP* mm, NodeP* bias) {
                *bias = nullptr;
                if (t->realized || t->dtype != n.dtype || t->shape != n.shape) return false;
                if (t->op == MATMUL) { *mm = t; return true; }
                if (t->op != ADD) return false;
                for (int k = 0; k < 2; ++k) {
                    const NodeP& m = t->in[k];
                    const NodeP& bv = t->in[1 - k];
                    if (m->op == MATMUL && !m->realized && m->dtype == n.dtype && m->shape == n.shape && m->in[1]->ndim() == 2 &&
                        bv->ndim() == 1 && bv->shape[0] == n.shape.back() && bv->dtype == n.dtype) {
                        *mm = m; *bias = bv;
                        return true;
                    }
                }
                return false;
            };
            NodeP gm, um;
            GateSpec spec;
            if (!product(act->in[0], &gm, &spec.bias_gate) || !product(up, &um, &spec.bias_up) || gm->in[0] != um->in[0]) continue;
            spec.b2 = um->in[1];
            spec.sigmoid = act->op == SIGMOID;
            bool fell_back = false;
            st = run_matmul(n, gm->in[0], gm->in[1], nullptr, &spec, &fell_back);
            if (st != MK_OK || !fell_back) return st;
            break;
        }
        if (a->op == SILU && !a->realized && a->shape == b->shape) {
            NodeP g, u;
            if ((st = dense(a->in[0], &g)) != MK_OK || (st = dense(b, &u)) != MK_OK) return st;
            void *pg, *pu, *py;
            if ((st = alloc_output(n)) != MK_OK) return st;
            if ((st = node_ptr(*g, &pg)) != MK_OK || (st = node_ptr(*u, &pu)) != MK_OK || (st = node_ptr(n, &py)) != MK_OK) return st;
            return mk_swiglu(n.dev, t_stream, n.dtype, pg, pu, py, n.numel());
        }
    }
    if (mul) {
        // mul(sigmoid(x), x) is silu(x), mul(sigmoid(g), u) the sigmoid-gated unit: one kernel either way
        // (tensor/src/test/unit/fusion.rs:50-56); the operands may come in either order
        for (int side = 0; side < 2; ++side) {
            const NodeP& sg = n.in[side];
            const NodeP& other = n.in[1 - side];
            if (sg->op != SIGMOID || sg->realized || sg->shape != other->shape || sg->dtype != n.dtype || other->dtype != n.dtype) continue;
            NodeP g, u;
            if ((st = dense(sg->in[0], &g)) != MK_OK || (st = alloc_output(n)) != MK_OK) return st;
            void *pg, *pu, *py;
            if ((st = node_ptr(*g, &pg)) != MK_OK || (st = node_ptr(n, &py)) != MK_OK) return st;
            if (sg->in[0] == other) return ew_silu(n.dev, raw(t_stream), n.dtype, pg, py, n.numel());
            if ((st = dense(other, &u)) != MK_OK || (st = node_ptr(*u, &pu)) != MK_OK) return st;
            return ew_glu(n.dev, raw(t_stream), n.dtype, pg, pu, py, n.numel());
        }
    }
    NodeP ad, bd;
    if ((st = dense(a, &ad)) != MK_OK || (st = dense(b, &bd)) != MK_OK) return st;
    void *pa, *pb, *py;
    if ((st = alloc_output(n)) != MK_OK) return st;
    if ((st = node_ptr(*ad, &pa)) != MK_OK || (st = node_ptr(*bd, &pb)) != MK_OK || (st = node_ptr(n, &py)) != MK_OK) return st;
    if (n.numel() == 0) return MK_OK;
    if (ad->numel() == bd->numel()) {
        if (mul) return ew_mul(n.dev, raw(t_stream), n.dtype, pa, pb, py, n.numel());
        return mk_add(n.dev, t_stream, n.dtype, pa, pb, py, n.numel());
    }
    // trailing-dimension broadcast of the smaller operand
    const bool a_big = ad->numel() > bd->numel();
    return ew_binary_bcast(n.dev, raw(t_stream), n.dtype, mul ? 1 : 0, a_big ? pa : pb, a_big ? pb : pa, py, n.numel(),
                           a_big ? bd->numel() : ad->numel());
}

mk_status realize(const NodeP& np) {
    Node& n = *np;
    if (n.realized) {
        // recorded by a plan that has not run yet: the buffer holds nothing (fine for that plan's own recording)
        if (!n.has_data() && n.plan_ran != t_plan_ran)
            return fail(MK_ERR_NOT_ALLOCATED, "realize: an input was recorded into a plan that has not been launched yet; it holds no data");
        return MK_OK;
    }
    if (n.dev->mock && n.op != VIEW) return fail(MK_ERR_CUDA, "realize: no CUDA device (mock devices run no kernels)");
    mk_status st = MK_OK;
    switch (n.op) {
        case LEAF:
            return fail(MK_ERR_INVALID, "realize: leaf tensor without data");
        case VIEW: {
            NodeP src = n.in[0];
            if (!n.perm.empty()) {
                // permute(0,2,1,3) of a fresh attention result: let attention store that layout
                static const int32_t kSwap[4] = {0, 2, 1, 3};
                if (src->op == SDPA && !src->realized && n.perm.size() == 4 && std::equal(n.perm.begin(), n.perm.end(), kSwap)) {
                    if ((st = run_sdpa(*src, true)) != MK_OK) return st;
                    src->realized = true;
                    src->plan_ran = t_plan_ran;
                    src->in.clear();
                }
                if ((st = realize(src)) != MK_OK) return st;
                n.buf = src->buf;
                n.offset = src->offset;
                n.strides.resize(n.perm.size());
                for (size_t i = 0; i < n.perm.size(); ++i) n.strides[i] = src->strides[n.perm[i]];
            } else {
                NodeP d;
                if ((st = dense(src, &d)) != MK_OK) return st;   // reshape needs dense data
                n.buf = d->buf;
                n.offset = d->offset;
                n.strides = contiguous_strides(n.shape);
            }
            break;
        }
        case MATMUL:
            st = run_matmul(n, n.in[0], n.in[1], nullptr);
            break;
        case SDPA:
            st = run_sdpa(n, false);
            break;
        case ADD:
        case MUL:
            st = run_binary(n);
            break;
        case RMSNORM: {
            NodeP x;
            if ((st = dense(n.in[0], &x)) != MK_OK || (st = alloc_output(n)) != MK_OK) return st;
            void *px, *py;
            if ((st = node_ptr(*x, &px)) != MK_OK || (st = node_ptr(n, &py)) != MK_OK) return st;
            const int64_t cols = x->shape.back();
            st = n.numel() ? mk_rms_norm(n.dev, t_stream, x->dtype, n.dtype, px, nullptr, py, x->numel() / cols, cols, n.eps) : MK_OK;
            break;
        }
        case ROPE: {
            // x [..., S, H, D] or [..., S, D]; cos/sin [.., S, 1, D/2] or [S, D/2] broadcast over batch and heads
            NodeP x, c, s;
            if ((st = dense(n.in[0], &x)) != MK_OK || (st = dense(n.in[1], &c)) != MK_OK || (st = dense(n.in[2], &s)) != MK_OK) return st;
            if ((st = alloc_output(n)) != MK_OK) return st;
            void *px, *pc, *ps, *py;
            if ((st = node_ptr(*x, &px)) != MK_OK || (st = node_ptr(*c, &pc)) != MK_OK || (st = node_ptr(*s, &ps)) != MK_OK ||
                (st = node_ptr(n, &py)) != MK_OK)
                return st;
            const int64_t D = x->shape.back();
            const int64_t rows = x->numel() / D;
            const int64_t rows_cs = c->numel() / (D / 2);
            const int64_t row_div = n.row_div;
            st = n.numel() ? mk_rope(n.dev, t_stream, n.dtype, px, (const float*)pc, (const float*)ps, py, rows, (int32_t)D, rows_cs, row_div,
                                     n.interleaved)
                           : MK_OK;
            break;
        }
        case SILU:
        case SIGMOID: {
            NodeP x;
            if ((st = dense(n.in[0], &x)) != MK_OK || (st = alloc_output(n)) != MK_OK) return st;
            void *px, *py;
            if ((st = node_ptr(*x, &px)) != MK_OK || (st = node_ptr(n, &py)) != MK_OK) return st;
            st = n.op == SILU ? ew_silu(n.dev, raw(t_stream), n.dtype, px, py, n.numel())
                              : ew_sigmoid(n.dev, raw(t_stream), n.dtype, px, py, n.numel());
            break;
        }
        case CAST: {
            // cast(rms_norm(x)) back to x's own 16-bit type: one kernel that normalises in f32 and
            // rounds once on store (the f32 intermediate of the reference's graph never touches memory)
            if (n.in[0]->op == RMSNORM && !n.in[0]->realized && n.dtype != MK_F32 && n.in[0]->in[0]->dtype == n.dtype) {
                const NodeP& rn = n.in[0];
                NodeP x;
                if ((st = dense(rn->in[0], &x)) != MK_OK || (st = alloc_output(n)) != MK_OK) return st;
                void *px, *py;
                if ((st = node_ptr(*x, &px)) != MK_OK || (st = node_ptr(n, &py)) != MK_OK) return st;
                const int64_t cols = x->shape.back();
                st = n.numel() ? mk_rms_norm(n.dev, t_stream, x->dtype, n.dtype, px, nullptr, py, x->numel() / cols, cols, rn->eps) : MK_OK;
                break;
            }
            NodeP x;
            if ((st = dense(n.in[0], &x)) != MK_OK || (st = alloc_output(n)) != MK_OK) return st;
            void *px, *py;
            if ((st = node_ptr(*x, &px)) != MK_OK || (st = node_ptr(n, &py)) != MK_OK) return st;
            st = n.numel() ? mk_cast(n.dev, t_stream, x->dtype, n.dtype, px, py, n.numel()) : MK_OK;
            break;
        }
    }
    if (st != MK_OK) return st;
    n.realized = true;
    n.plan_ran = t_plan_ran;
    n.in.clear();   // a realized tensor is a buffer; its producers can go back to the cache
    return MK_OK;
}

NodeP make_cast(const NodeP& x, int32_t dtype) {
    if (x->dtype == dtype) return x;
    auto c = std::make_shared<Node>();
    c->op = CAST;
    c->dev = x->dev;
    c->dtype = dtype;
    c->shape = x->shape;
    c->in = {x};
    return c;
}

}  // namespace

struct mk_tensor {
    NodeP node;
};

struct mk_plan {
    std::shared_ptr<std::atomic<bool>> ran = std::make_shared<std::atomic<bool>>(false);   // set by the first launch
    mk_device* dev = nullptr;
    mk_stream capture{nullptr, nullptr};              // the stream the plan was recorded on
    cudaGraphExec_t exec = nullptr;
    std::vector<std::shared_ptr<mk_buf>> retained;   // every buffer the recorded kernels read or write
    NodeP result;
    int32_t kernels = 0;
};

namespace {
mk_tensor* wrap(const NodeP& n) { return new mk_tensor{n}; }

NodeP new_node(Op op, const NodeP& like, std::vector<NodeP> in) {
    auto n = std::make_shared<Node>();
    n->op = op;
    n->dev = like->dev;
    n->dtype = like->dtype;
    n->shape = like->shape;
    n->in = std::move(in);
    return n;
}
}  // namespace

extern "C" {

mk_status mk_tensor_from_bytes(mk_device* dev, const void* data, int32_t dtype, const int64_t* shape, int32_t ndim, mk_tensor** out) {
    MK_REQUIRE(dev && out && (shape || ndim == 0), "mk_tensor_from_bytes: null argument");
    MK_REQUIRE(dtype_valid(dtype) || dtype == MK_BOOL, "mk_tensor_from_bytes: unknown dtype %d", dtype);
    MK_REQUIRE(ndim >= 0 && ndim <= MK_MAX_DIMS, "mk_tensor_from_bytes: ndim %d out of range", ndim);
    auto n = std::make_shared<Node>();
    n->op = LEAF;
    n->dev = dev;
    n->dtype = dtype;
    n->shape.assign(shape, shape + ndim);
    for (auto d : n->shape) MK_REQUIRE(d >= 0, "mk_tensor_from_bytes: negative dimension");
    MK_REQUIRE(data || n->numel() == 0, "mk_tensor_from_bytes: null data");
    if (!dev->mock) MK_CUDA(cudaSetDevice(dev->ordinal));
    mk_status st = alloc_output(*n);
    if (st != MK_OK) return st;
    if (n->numel() > 0) {
        st = mk_copy_h2d(n->buf.get(), data, (size_t)n->numel() * dtype_size(dtype), nullptr);
        if (st != MK_OK) return st;
        // the caller may reuse its memory as soon as this returns
        if (!dev->mock) MK_CUDA(cudaStreamSynchronize(0));
    }
    n->realized = true;
    *out = wrap(n);
    return MK_OK;
}

mk_status mk_tensor_free(mk_tensor* t) {
    MK_REQUIRE(t, "mk_tensor_free: null tensor");
    delete t;
    return MK_OK;
}

mk_status mk_tensor_shape(mk_tensor* t, int64_t* shape, int32_t* ndim, int32_t* dtype) {
    MK_REQUIRE(t && ndim, "mk_tensor_shape: null argument");
    const Node& n = *t->node;
    *ndim = n.ndim();
    if (shape)
        for (int i = 0; i < n.ndim(); ++i) shape[i] = n.shape[i];
    if (dtype) *dtype = n.dtype;
    return MK_OK;
}

mk_status mk_tensor_matmul(mk_tensor* at, mk_tensor* bt, mk_tensor** out) {
    MK_REQUIRE(at && bt && out, "mk_tensor_matmul: null argument");
    NodeP a = at->node, b = bt->node;
    // tensor/src/matmul.rs:84-92: both operands need >= 1 dimension and matching contraction sizes
    MK_REQUIRE(a->ndim() >= 1 && b->ndim() >= 1, "matmul: 0-dimensional operand (lhs %dD, rhs %dD)", a->ndim(), b->ndim());
    const int64_t K = a->shape.back();
    const int64_t Kb = b->ndim() == 1 ? b->shape[0] : b->shape[b->ndim() - 2];
    MK_REQUIRE(K == Kb, "matmul: shape mismatch, lhs [..., %lld] vs rhs contraction %lld", (long long)K, (long long)Kb);
    MK_REQUIRE(a->dev == b->dev, "matmul: operands live on different devices");
    int32_t dt = a->dtype;
    if (a->dtype != b->dtype) dt = MK_F32;   // least upper dtype of (bf16|f16, f32) and (bf16, f16)
    a = make_cast(a, dt);
    b = make_cast(b, dt);
    auto n = std::make_shared<Node>();
    n->op = MATMUL;
    n->dev = a->dev;
    n->dtype = dt;
    // result shape: a[..., M] + b[..., N] with the 1-D rules of tensor/src/matmul.rs:95-109
    std::vector<int64_t> lead;
    if (b->ndim() > 2) lead.assign(b->shape.begin(), b->shape.end() - 2);
    else if (a->ndim() > 2) lead.assign(a->shape.begin(), a->shape.end() - 2);
    n->shape = lead;
    if (a->ndim() >= 2) n->shape.push_back(a->shape[a->ndim() - 2]);
    if (b->ndim() >= 2) n->shape.push_back(b->shape.back());
    n->in = {a, b};
    *out = wrap(n);
    return MK_OK;
}

mk_status mk_tensor_sdpa(mk_tensor* qt, mk_tensor* kt, mk_tensor* vt, mk_tensor* maskt, float scale, int32_t causal, float softcap,
                         mk_tensor** out) {
    MK_REQUIRE(qt && kt && vt && out, "mk_tensor_sdpa: null argument");
    NodeP q = qt->node, k = kt->node, v = vt->node;
    MK_REQUIRE(q->ndim() == 4 && k->ndim() == 4 && v->ndim() == 4, "scaled_dot_product_attention: Q, K, V must be [B,H,S,D]");
    MK_REQUIRE(q->dtype == k->dtype && q->dtype == v->dtype, "scaled_dot_product_attention: dtype mismatch");
    MK_REQUIRE(q->shape[0] == k->shape[0] && k->shape[0] == v->shape[0], "scaled_dot_product_attention: batch mismatch");
    MK_REQUIRE(q->shape[3] == k->shape[3], "scaled_dot_product_attention: head size mismatch (%lld vs %lld)", (long long)q->shape[3],
               (long long)k->shape[3]);
    MK_REQUIRE(k->shape[1] == v->shape[1] && k->shape[2] == v->shape[2], "scaled_dot_product_attention: K/V shape mismatch");
    MK_REQUIRE(k->shape[1] > 0 && q->shape[1] % k->shape[1] == 0, "scaled_dot_product_attention: query heads must be a multiple of kv heads");
    auto n = std::make_shared<Node>();
    n->op = SDPA;
    n->dev = q->dev;
    n->dtype = q->dtype;
    n->shape = {q->shape[0], q->shape[1], q->shape[2], v->shape[3]};
    n->scale = scale; n->causal = causal; n->softcap = softcap;
    n->in = {q, k, v};
    if (maskt) {
        NodeP m = maskt->node;
        MK_REQUIRE(m->ndim() >= 2 && m->ndim() <= 4, "scaled_dot_product_attention: the mask needs 2 to 4 dimensions, got %d", m->ndim());
        MK_REQUIRE(m->shape.back() == k->shape[2], "scaled_dot_product_attention: the mask's last dimension must be Sk = %lld", (long long)k->shape[2]);
        const int64_t want[3] = {q->shape[0], q->shape[1], q->shape[2]};      // B, H, Sq
        for (int j = 0; j < m->ndim() - 1; ++j) {
            const int64_t w = want[3 - (m->ndim() - 1) + j];
            MK_REQUIRE(m->shape[j] == 1 || m->shape[j] == w, "scaled_dot_product_attention: mask dimension %d is %lld, expected 1 or %lld", j,
                       (long long)m->shape[j], (long long)w);
        }
        n->in.push_back(m->dtype == MK_BOOL ? m : make_cast(m, MK_F32));     // bool: true attends; anything else is added as f32
    }
    *out = wrap(n);
    return MK_OK;
}

mk_status mk_tensor_rms_norm(mk_tensor* xt, float eps, mk_tensor** out) {
    MK_REQUIRE(xt && out, "mk_tensor_rms_norm: null argument");
    NodeP x = xt->node;
    MK_REQUIRE(x->ndim() >= 1 && x->shape.back() > 0, "rms_norm: needs a non-empty last axis");
    NodeP n = new_node(RMSNORM, x, {x});
    n->dtype = MK_F32;   // self * rsqrt(f32) promotes (tensor/src/nn/norm.rs:98-109)
    n->eps = eps;
    *out = wrap(n);
    return MK_OK;
}

mk_status mk_tensor_rope(mk_tensor* xt, mk_tensor* ct, mk_tensor* st_, int32_t interleaved, mk_tensor** out) {
    MK_REQUIRE(xt && ct && st_ && out, "mk_tensor_rope: null argument");
    NodeP x = xt->node, c = ct->node, s = st_->node;
    MK_REQUIRE(x->ndim() >= 1 && x->shape.back() % 2 == 0, "apply_rotary_emb: last dim must be even");
    const int64_t half = x->shape.back() / 2;
    MK_REQUIRE(c->ndim() >= 1 && c->shape.back() == half && s->shape == c->shape, "apply_rotary_emb: cos/sin must be [..., D/2]");
    // cos/sin broadcast against x (right-aligned, last axis aside).  Supported pattern: a run of axes
    // equal to x's, size-1 axes around it -- e.g. [1,S,1,D/2] against [B,S,H,D], or [S,D/2] against
    // [B,H,S,D].  Input rows after the run (the heads) share one table row.
    MK_REQUIRE(c->ndim() <= x->ndim(), "apply_rotary_emb: cos/sin have more dimensions than the input");
    int64_t row_div = 1;
    int state = 0;   // 0: trailing ones, 1: inside the run, 2: leading ones
    for (int i = 1; i < c->ndim(); ++i) {
        const int64_t cd = c->shape[c->ndim() - 1 - i], xd = x->shape[x->ndim() - 1 - i];
        if (cd == 1 && xd != 1) {
            if (state == 0) row_div *= xd;
            else state = 2;
        } else {
            MK_REQUIRE(cd == xd && state != 2, "apply_rotary_emb: cos/sin do not broadcast to the input");
            state = 1;
        }
    }
    NodeP n = new_node(ROPE, x, {x, make_cast(c, MK_F32), make_cast(s, MK_F32)});
    n->interleaved = interleaved;
    n->row_div = row_div;
    *out = wrap(n);
    return MK_OK;
}

mk_status mk_tensor_silu(mk_tensor* xt, mk_tensor** out) {
    MK_REQUIRE(xt && out, "mk_tensor_silu: null argument");
    *out = wrap(new_node(SILU, xt->node, {xt->node}));
    return MK_OK;
}

mk_status mk_tensor_sigmoid(mk_tensor* xt, mk_tensor** out) {
    MK_REQUIRE(xt && out, "mk_tensor_sigmoid: null argument");
    *out = wrap(new_node(SIGMOID, xt->node, {xt->node}));
    return MK_OK;
}

static mk_status binary(Op op, mk_tensor* at, mk_tensor* bt, mk_tensor** out, const char* who) {
    MK_REQUIRE(at && bt && out, "%s: null argument", who);
    NodeP a = at->node, b = bt->node;
    const int32_t dt = a->dtype == b->dtype ? a->dtype : MK_F32;
    a = make_cast(a, dt);
    b = make_cast(b, dt);
    // same shape, or one operand equals the trailing dimensions of the other
    const NodeP& big = a->numel() >= b->numel() ? a : b;
    const NodeP& small = a->numel() >= b->numel() ? b : a;
    bool ok = small->ndim() <= big->ndim();
    for (int i = 0; ok && i < small->ndim(); ++i) ok = small->shape[small->ndim() - 1 - i] == big->shape[big->ndim() - 1 - i];
    ok = ok || small->numel() == 1;    // a one-element tensor scales / shifts everything (Tensor::gemm's alpha and beta)
    MK_REQUIRE(ok, "%s: shapes do not broadcast (only trailing-dimension and one-element broadcast are supported)", who);
    NodeP n = new_node(op, big, {a, b});
    n->dtype = dt;
    *out = wrap(n);
    return MK_OK;
}

mk_status mk_tensor_add(mk_tensor* a, mk_tensor* b, mk_tensor** out) { return binary(ADD, a, b, out, "add"); }
mk_status mk_tensor_mul(mk_tensor* a, mk_tensor* b, mk_tensor** out) { return binary(MUL, a, b, out, "mul"); }

mk_status mk_tensor_cast(mk_tensor* xt, int32_t dtype, mk_tensor** out) {
    MK_REQUIRE(xt && out, "mk_tensor_cast: null argument");
    MK_REQUIRE(dtype_valid(dtype), "mk_tensor_cast: unknown dtype %d", dtype);
    *out = wrap(make_cast(xt->node, dtype));
    return MK_OK;
}

mk_status mk_tensor_reshape(mk_tensor* xt, const int64_t* shape, int32_t ndim, mk_tensor** out) {
    MK_REQUIRE(xt && out && (shape || ndim == 0), "mk_tensor_reshape: null argument");
    MK_REQUIRE(ndim >= 0 && ndim <= MK_MAX_DIMS, "mk_tensor_reshape: ndim %d out of range", ndim);
    NodeP x = xt->node;
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) {
        MK_REQUIRE(shape[i] >= 0, "mk_tensor_reshape: negative dimension");
        n *= shape[i];
    }
    MK_REQUIRE(n == x->numel(), "reshape: %lld elements into a shape of %lld", (long long)x->numel(), (long long)n);
    NodeP v = new_node(VIEW, x, {x});
    v->shape.assign(shape, shape + ndim);
    *out = wrap(v);
    return MK_OK;
}

mk_status mk_tensor_permute(mk_tensor* xt, const int32_t* axes, int32_t ndim, mk_tensor** out) {
    MK_REQUIRE(xt && axes && out, "mk_tensor_permute: null argument");
    NodeP x = xt->node;
    MK_REQUIRE(ndim == x->ndim(), "permute: %d axes for a %d-dimensional tensor", ndim, x->ndim());
    std::vector<bool> seen(ndim, false);
    for (int i = 0; i < ndim; ++i) {
        MK_REQUIRE(axes[i] >= 0 && axes[i] < ndim && !seen[axes[i]], "permute: axes are not a permutation");
        seen[axes[i]] = true;
    }
    NodeP v = new_node(VIEW, x, {x});
    v->perm.assign(axes, axes + ndim);
    for (int i = 0; i < ndim; ++i) v->shape[i] = x->shape[axes[i]];
    *out = wrap(v);
    return MK_OK;
}

mk_status mk_tensor_realize(mk_tensor* t) {
    MK_REQUIRE(t, "mk_tensor_realize: null tensor");
    Node& n = *t->node;
    const uint64_t before = n.dev->launches.load();
    AllocStreamScope scope(raw(t_stream));      // buffers taken from the cache are ordered on the realising stream
    mk_status st = realize(t->node);
    n.last_launches = (int32_t)(n.dev->launches.load() - before);
    return st;
}

mk_status mk_tensor_last_launches(mk_tensor* t, int32_t* launches) {
    MK_REQUIRE(t && launches, "mk_tensor_last_launches: null argument");
    *launches = t->node->last_launches;
    return MK_OK;
}

mk_status mk_tensor_copyout(mk_tensor* t, void* dst, size_t bytes) {
    MK_REQUIRE(t && (dst || bytes == 0), "mk_tensor_copyout: null argument");
    NodeP n = t->node;
    if (!n->realized) return fail(MK_ERR_NOT_ALLOCATED, "as_vec: tensor is not realized; call realize() first");
    if (!n->has_data()) return fail(MK_ERR_NOT_ALLOCATED, "as_vec: the tensor was recorded into a plan that has not been launched yet");
    const size_t want = (size_t)n->numel() * dtype_size(n->dtype);
    if (bytes != want) return fail(MK_ERR_SIZE_MISMATCH, "as_vec: %zu bytes requested, tensor holds %zu", bytes, want);
    if (want == 0) return MK_OK;
    NodeP d;
    mk_status st = dense(n, &d);
    if (st != MK_OK) return st;
    void* p;
    if ((st = node_ptr(*d, &p)) != MK_OK) return st;
    if (n->dev->mock) {
        memcpy(dst, p, want);
        return MK_OK;
    }
    MK_CUDA(cudaMemcpy(dst, p, want, cudaMemcpyDeviceToHost));
    return MK_OK;
}

// ---- plans: record once, replay many times ---------------------------------------------------------------
// The reference prepares an ExecutionPlan once and executes it repeatedly
// (runtime/src/execution_plan.rs:88-106, 168-181).  Here the kernels that realising a tensor launches are
// recorded into a CUDA graph by stream capture; replaying the plan costs one launch call instead of one
// per kernel.  Leaf tensors are read at their addresses, so writing new data into them
// (mk_tensor_write) and replaying computes the same graph on the new data.
mk_status mk_tensor_compile(mk_tensor* t, mk_plan** out) {
    MK_REQUIRE(t && out, "mk_tensor_compile: null argument");
    NodeP n = t->node;
    mk_device* dev = n->dev;
    if (dev->mock) return fail(MK_ERR_CUDA, "mk_tensor_compile: no CUDA device (mock devices run no kernels)");
    if (n->realized) return fail(MK_ERR_INVALID, "mk_tensor_compile: the tensor is already realized; there is nothing to record");
    MK_CUDA(cudaSetDevice(dev->ordinal));
    auto plan = new mk_plan();
    plan->dev = dev;
    cudaError_t e = cudaStreamCreateWithFlags(&plan->capture.s, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete plan;
        return fail(MK_ERR_CUDA, "mk_tensor_compile: %s", cudaGetErrorString(e));
    }
    plan->capture.dev = dev;
    // relaxed mode: the allocator may have to call cudaMalloc for a size it has not cached yet
    e = cudaStreamBeginCapture(plan->capture.s, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) {
        cudaStreamDestroy(plan->capture.s);
        delete plan;
        return fail(MK_ERR_CUDA, "mk_tensor_compile: %s", cudaGetErrorString(e));
    }
    mark_plan_stream(dev, plan->capture.s);     // own error word and claim counter for the plan's kernels
    t_stream = &plan->capture;
    t_retain = &plan->retained;
    t_plan_ran = plan->ran;
    const uint64_t before = dev->launches.load();
    mk_status st;
    {
        AllocStreamScope scope(plan->capture.s);
        st = realize(n);
    }
    t_stream = nullptr;
    t_retain = nullptr;
    t_plan_ran.reset();
    cudaGraph_t graph = nullptr;
    e = cudaStreamEndCapture(plan->capture.s, &graph);
    if (st == MK_OK && e != cudaSuccess) st = fail(MK_ERR_CUDA, "mk_tensor_compile: capture failed: %s", cudaGetErrorString(e));
    if (st == MK_OK) {
        e = cudaGraphInstantiate(&plan->exec, graph, 0);
        if (e != cudaSuccess) st = fail(MK_ERR_CUDA, "mk_tensor_compile: %s", cudaGetErrorString(e));
    }
    if (graph) cudaGraphDestroy(graph);
    if (st != MK_OK) {
        cudaGetLastError();
        mk_plan_free(plan);
        return st;
    }
    plan->kernels = (int32_t)(dev->launches.load() - before);
    dev->launches -= (uint64_t)plan->kernels;     // recorded, not run: launches are counted when the plan is replayed
    n->last_launches = plan->kernels;
    plan->result = n;
    *out = plan;
    return MK_OK;
}

mk_status mk_plan_launch(mk_plan* plan, mk_stream* s) {
    MK_REQUIRE(plan && plan->exec, "mk_plan_launch: null plan");
    MK_CUDA(cudaSetDevice(plan->dev->ordinal));
    MK_CUDA(cudaGraphLaunch(plan->exec, raw(s)));
    touch_stream(plan->dev, raw(s));
    plan->ran->store(true);
    plan->dev->launches += (uint64_t)plan->kernels;
    return MK_OK;
}

mk_status mk_plan_kernel_count(mk_plan* plan, int32_t* kernels) {
    MK_REQUIRE(plan && kernels, "mk_plan_kernel_count: null argument");
    *kernels = plan->kernels;
    return MK_OK;
}

mk_status mk_plan_free(mk_plan* plan) {
    if (!plan) return MK_OK;
    if (plan->exec) cudaGraphExecDestroy(plan->exec);
    if (plan->capture.s) {
        release_stream_state(plan->dev, plan->capture.s);     // scratch, error word and claim counter of the recorded kernels
        cudaStreamDestroy(plan->capture.s);
    }
    delete plan;     // releases the retained buffers to the allocator cache
    return MK_OK;
}

mk_status mk_tensor_write(mk_tensor* t, const void* data, size_t bytes) {
    MK_REQUIRE(t && (data || bytes == 0), "mk_tensor_write: null argument");
    Node& n = *t->node;
    if (!n.realized) return fail(MK_ERR_NOT_ALLOCATED, "mk_tensor_write: the tensor has no buffer yet (not realized)");
    if (n.offset != 0 || !is_contiguous(n)) return fail(MK_ERR_UNSUPPORTED, "mk_tensor_write: the tensor is a view; write to the tensor that owns the data");
    const size_t want = (size_t)n.numel() * dtype_size(n.dtype);
    if (bytes != want) return fail(MK_ERR_SIZE_MISMATCH, "mk_tensor_write: %zu bytes given, tensor holds %zu", bytes, want);
    if (want == 0) return MK_OK;
    return mk_copy_h2d(n.buf.get(), data, want, nullptr);
}

}  // extern "C"
