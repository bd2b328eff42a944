#include "Layers.h"

#include <stdexcept>
#include <type_traits>

#include "tt_attn.h"

namespace {

void raise(int rc, const char* who) {
    if (rc == TT_OK) return;
    std::string msg = std::string(who) + ": " + tt_last_error();
    if (rc == TT_ERR_NULL || rc == TT_ERR_BAD_SHAPE || rc == TT_ERR_BAD_DTYPE || rc == TT_ERR_WORKSPACE)
        throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

template <typename T>
void require_gpu(const TinyTensor<T>& t, const char* who, const char* name) {
    if (t.device != "gpu")
        throw std::invalid_argument(std::string(who) + ": tensor '" + name + "' is on '" + t.device +
                                    "'; attention runs on gpu tensors only");
}

template <typename T>
tt_attn_desc describe(const TinyTensor<T>& q, const TinyTensor<T>& k, const TinyTensor<T>& v, bool causal, float scale,
                      const char* who) {
    if (q.shape.size() != 4 || k.shape.size() != 4 || v.shape.size() != 4)
        throw std::invalid_argument(std::string(who) + ": q, k, v must be 4-D [B,H,rows,D]");
    if (k.shape != v.shape || q.shape[0] != k.shape[0] || k.shape[1] < 1 || q.shape[1] % k.shape[1] != 0 ||
        q.shape[3] != k.shape[3])
        throw std::invalid_argument(std::string(who) + ": q, k, v shapes do not agree (k, v heads must divide q heads)");
    tt_attn_desc d;
    d.Hkv = k.shape[1];   // fewer key/value heads than query heads: grouped attention
    d.B = q.shape[0];
    d.H = q.shape[1];
    d.S = q.shape[2];
    d.L = k.shape[2];
    d.D = q.shape[3];
    d.dtype = std::is_same<T, float>::value ? TT_F32 : TT_BF16;
    d.causal = causal ? 1 : 0;
    d.scale = scale;
    return d;
}

struct PoolBuffer {   // workspace taken from the pooled allocator for the duration of a call
    void* p = nullptr;
    size_t bytes = 0;
    explicit PoolBuffer(size_t n) : bytes(n) {
        if (n) raise(tt_alloc(n, &p), "workspace");
    }
    ~PoolBuffer() { tt_free(p); }
};

}  // namespace

template <typename T>
void AttentionForward(const TinyTensor<T>& q, const TinyTensor<T>& k, const TinyTensor<T>& v, TinyTensor<T>& out,
                      TinyTensor<float>& lse, bool causal, float scale) {
    const char* who = "AttentionForward";
    require_gpu(q, who, "q"); require_gpu(k, who, "k"); require_gpu(v, who, "v");
    tt_attn_desc d = describe(q, k, v, causal, scale, who);
    if (out.device != "gpu") out.gpu();
    if (lse.device != "gpu") lse.gpu();
    out.resize(q.shape);
    lse.resize({d.B, d.H, d.S});
    int rc;
    if (d.S == 1 && d.dtype == TT_BF16) {
        tt_attn_desc dd = d;
        dd.causal = 0;
        PoolBuffer ws(tt_attn_decode_workspace_bytes(&dd));
        rc = tt_attn_decode(&dd, q.p_data, k.p_data, v.p_data, out.p_data, lse.p_data, ws.p, ws.bytes, nullptr);
        if (rc == TT_OK) rc = tt_check_device_status(nullptr);   // synchronises before the workspace is returned
    } else {
        rc = tt_attn_fwd(&d, q.p_data, k.p_data, v.p_data, out.p_data, lse.p_data, nullptr);
        if (rc == TT_OK) rc = tt_check_device_status(nullptr);   // "returns when done", like the reference's ops
    }
    raise(rc, who);
}

template <typename T>
void AttentionBackward(const TinyTensor<T>& q, const TinyTensor<T>& k, const TinyTensor<T>& v,
                       const TinyTensor<T>& out, const TinyTensor<float>& lse, TinyTensor<T>& grad_q,
                       TinyTensor<T>& grad_k, TinyTensor<T>& grad_v, const TinyTensor<T>& grad_out, bool causal,
                       float scale) {
    const char* who = "AttentionBackward";
    require_gpu(q, who, "q"); require_gpu(k, who, "k"); require_gpu(v, who, "v");
    require_gpu(out, who, "out"); require_gpu(lse, who, "lse"); require_gpu(grad_out, who, "grad_out");
    tt_attn_desc d = describe(q, k, v, causal, scale, who);
    if (out.shape != q.shape || grad_out.shape != q.shape)
        throw std::invalid_argument(std::string(who) + ": out and grad_out must have q's shape");
    if (lse.size != (size_t)d.B * d.H * d.S) throw std::invalid_argument(std::string(who) + ": lse must be [B,H,S]");
    for (TinyTensor<T>* g : {&grad_q, &grad_k, &grad_v})
        if (g->device != "gpu") g->gpu();
    grad_q.resize(q.shape);
    grad_k.resize(k.shape);
    grad_v.resize(v.shape);
    PoolBuffer ws(tt_attn_bwd_workspace_bytes(&d));
    int rc = tt_attn_bwd(&d, q.p_data, k.p_data, v.p_data, out.p_data, lse.p_data, grad_out.p_data, grad_q.p_data,
                         grad_k.p_data, grad_v.p_data, ws.p, ws.bytes, nullptr);
    if (rc == TT_OK) rc = tt_check_device_status(nullptr);
    raise(rc, who);
}

template <typename T>
void SoftmaxForward(const TinyTensor<T>& input, TinyTensor<T>& output) {
    require_gpu(input, "SoftmaxForward", "input");
    if (input.shape.empty()) throw std::invalid_argument("SoftmaxForward: empty shape");
    if (output.device != "gpu") output.gpu();
    output.resize(input.shape);
    const int cols = input.shape.back();
    const long long rows = cols ? (long long)(input.size / (size_t)cols) : 0;
    int rc = tt_softmax_fwd(input.p_data, output.p_data, rows, cols, std::is_same<T, float>::value ? TT_F32 : TT_BF16, nullptr);
    if (rc == TT_OK) rc = tt_check_device_status(nullptr);
    raise(rc, "SoftmaxForward");
}

template <typename T>
void SoftmaxBackward(const TinyTensor<T>& output, const TinyTensor<T>& grad_output, TinyTensor<T>& grad_input) {
    require_gpu(output, "SoftmaxBackward", "output");
    require_gpu(grad_output, "SoftmaxBackward", "grad_output");
    if (output.shape.empty() || output.shape != grad_output.shape)
        throw std::invalid_argument("SoftmaxBackward: output and grad_output must have one shape");
    if (grad_input.device != "gpu") grad_input.gpu();
    grad_input.resize(output.shape);
    const int cols = output.shape.back();
    const long long rows = cols ? (long long)(output.size / (size_t)cols) : 0;
    int rc = tt_softmax_bwd(output.p_data, grad_output.p_data, grad_input.p_data, rows, cols,
                            std::is_same<T, float>::value ? TT_F32 : TT_BF16, nullptr);
    if (rc == TT_OK) rc = tt_check_device_status(nullptr);
    raise(rc, "SoftmaxBackward");
}

namespace {
template <typename T>
void fc_dims(const TinyTensor<T>& input, const TinyTensor<T>& weight, const TinyTensor<T>& bias, const char* who,
             long long& rows, int& fin, int& fout, bool& scalar_bias) {
    require_gpu(input, who, "input"); require_gpu(weight, who, "weight"); require_gpu(bias, who, "bias");
    if (input.shape.empty() || weight.shape.size() != 2 || input.shape.back() != weight.shape[0])
        throw std::invalid_argument(std::string(who) + ": input [..., in] and weight [in, out] do not agree");
    fin = weight.shape[0];
    fout = weight.shape[1];
    rows = fin ? (long long)(input.size / (size_t)fin) : 0;
    scalar_bias = bias.shape.size() == 1 && bias.shape[0] == 1 && fout != 1;
    if (!scalar_bias && bias.size != (size_t)fout)
        throw std::invalid_argument(std::string(who) + ": bias must hold out_features values or one value");
}
}  // namespace

template <typename T>
void FcForward(const TinyTensor<T>& input, TinyTensor<T>& output, const TinyTensor<T>& weight, const TinyTensor<T>& bias) {
    const char* who = "FcForward";
    long long rows; int fin, fout; bool scalar_bias;
    fc_dims(input, weight, bias, who, rows, fin, fout, scalar_bias);
    std::vector<int> oshape(input.shape.begin(), input.shape.end() - 1);
    oshape.push_back(fout);
    if (output.device != "gpu") output.gpu();
    output.resize(oshape);
    const int dt = std::is_same<T, float>::value ? TT_F32 : TT_BF16;
    int rc;
    if (scalar_bias) {   // one value for every output: spread it, as the reference does (src/Layers.cu:29-34)
        TinyTensor<T> b1(bias);
        TinyTensor<T> full(std::vector<int>{fout}, "gpu");
        full.floatks(b1.get_data_f32()[0]);
        rc = tt_fc_fwd(input.p_data, weight.p_data, full.p_data, output.p_data, rows, fin, fout, dt, nullptr);
        if (rc == TT_OK) rc = tt_check_device_status(nullptr);   // `full` must outlive the kernel
    } else {
        rc = tt_fc_fwd(input.p_data, weight.p_data, bias.p_data, output.p_data, rows, fin, fout, dt, nullptr);
        if (rc == TT_OK) rc = tt_check_device_status(nullptr);
    }
    raise(rc, who);
}

template <typename T>
void FcBackward(const TinyTensor<T>& input, const TinyTensor<T>& /*output*/, const TinyTensor<T>& weight,
                const TinyTensor<T>& bias, TinyTensor<T>& grad_input, const TinyTensor<T>& grad_output,
                TinyTensor<T>& grad_weight, TinyTensor<T>& grad_bias) {
    const char* who = "FcBackward";
    long long rows; int fin, fout; bool scalar_bias;
    fc_dims(input, weight, bias, who, rows, fin, fout, scalar_bias);
    require_gpu(grad_output, who, "grad_output");
    if (grad_output.size != (size_t)rows * (size_t)fout)
        throw std::invalid_argument(std::string(who) + ": grad_output does not match [rows, out_features]");
    for (TinyTensor<T>* t : {&grad_input, &grad_weight, &grad_bias})
        if (t->device != "gpu") t->gpu();
    grad_input.resize(input.shape);
    grad_weight.resize(weight.shape);
    grad_bias.resize(bias.shape);
    const int dt = std::is_same<T, float>::value ? TT_F32 : TT_BF16;
    PoolBuffer ws(tt_fc_bwd_workspace_bytes(rows, fin, fout, dt));
    int rc = tt_fc_bwd(input.p_data, weight.p_data, grad_output.p_data, grad_input.p_data, grad_weight.p_data,
                       grad_bias.p_data, scalar_bias ? 1 : 0, rows, fin, fout, dt, ws.p, ws.bytes, nullptr);
    if (rc == TT_OK) rc = tt_check_device_status(nullptr);
    raise(rc, who);
}

#define TT_INSTANTIATE_FC(T)                                                                                          \
    template void FcForward<T>(const TinyTensor<T>&, TinyTensor<T>&, const TinyTensor<T>&, const TinyTensor<T>&);      \
    template void FcBackward<T>(const TinyTensor<T>&, const TinyTensor<T>&, const TinyTensor<T>&, const TinyTensor<T>&, \
                                TinyTensor<T>&, const TinyTensor<T>&, TinyTensor<T>&, TinyTensor<T>&);
TT_INSTANTIATE_FC(float)
TT_INSTANTIATE_FC(__nv_bfloat16)
#undef TT_INSTANTIATE_FC

template void AttentionForward<float>(const TinyTensor<float>&, const TinyTensor<float>&, const TinyTensor<float>&,
                                      TinyTensor<float>&, TinyTensor<float>&, bool, float);
template void AttentionForward<__nv_bfloat16>(const TinyTensor<__nv_bfloat16>&, const TinyTensor<__nv_bfloat16>&,
                                              const TinyTensor<__nv_bfloat16>&, TinyTensor<__nv_bfloat16>&,
                                              TinyTensor<float>&, bool, float);
template void AttentionBackward<float>(const TinyTensor<float>&, const TinyTensor<float>&, const TinyTensor<float>&,
                                       const TinyTensor<float>&, const TinyTensor<float>&, TinyTensor<float>&,
                                       TinyTensor<float>&, TinyTensor<float>&, const TinyTensor<float>&, bool, float);
template void AttentionBackward<__nv_bfloat16>(const TinyTensor<__nv_bfloat16>&, const TinyTensor<__nv_bfloat16>&,
                                               const TinyTensor<__nv_bfloat16>&, const TinyTensor<__nv_bfloat16>&,
                                               const TinyTensor<float>&, TinyTensor<__nv_bfloat16>&,
                                               TinyTensor<__nv_bfloat16>&, TinyTensor<__nv_bfloat16>&,
                                               const TinyTensor<__nv_bfloat16>&, bool, float);
template void SoftmaxForward<float>(const TinyTensor<float>&, TinyTensor<float>&);
template void SoftmaxBackward<float>(const TinyTensor<float>&, const TinyTensor<float>&, TinyTensor<float>&);
