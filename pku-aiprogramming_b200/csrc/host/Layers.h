// Operator layer in the reference's style (src/Layers.h:8-99 of the reference project): free
// function templates over TinyTensor that resize their outputs and return when the work is
// done.  The attention path and its neighbours live here (row softmax, the fully connected layer of
// the projections either side of attention); the reference's Conv/Pool/CrossEntropy layers are a
// different workload and are not part of this library.
#ifndef TT_HOST_LAYERS_H
#define TT_HOST_LAYERS_H

#include "TinyTensor.h"

// out = softmax(scale * q k^T [+ causal mask]) v        q,out [B,H,S,D]   k,v [B,H,L,D]
// lse [B,H,S] = log of the softmax denominator (kept for the backward).
// scale <= 0 selects 1/sqrt(D).  Tensors must be on "gpu": there is no CPU implementation.
// T = float (exact fp32 kernels) or __nv_bfloat16 (tensor-core kernels; S == 1 takes the
// split-KV decode kernel).
template <typename T>
void AttentionForward(const TinyTensor<T>& q, const TinyTensor<T>& k, const TinyTensor<T>& v, TinyTensor<T>& out,
                      TinyTensor<float>& lse, bool causal, float scale);

// grad_q, grad_k, grad_v of sum(out * grad_out); out and lse come from AttentionForward.
template <typename T>
void AttentionBackward(const TinyTensor<T>& q, const TinyTensor<T>& k, const TinyTensor<T>& v,
                       const TinyTensor<T>& out, const TinyTensor<float>& lse, TinyTensor<T>& grad_q,
                       TinyTensor<T>& grad_k, TinyTensor<T>& grad_v, const TinyTensor<T>& grad_out, bool causal,
                       float scale);

// Softmax over the last axis, all leading axes flattened to rows, row maximum subtracted:
// the semantics of the reference's SoftmaxForward (src/Layers.cu:324-349), in one kernel.
template <typename T>
void SoftmaxForward(const TinyTensor<T>& input, TinyTensor<T>& output);

// grad_input = output * (grad_output - rowsum(grad_output * output)) for output = softmax(input).
template <typename T>
void SoftmaxBackward(const TinyTensor<T>& output, const TinyTensor<T>& grad_output, TinyTensor<T>& grad_input);

// output[..., out] = input[..., in] . weight[in, out] + bias, bias of shape [out] or [1] (one value
// for every output) -- signature and semantics of the reference's FcForward (src/Layers.cu:9-40).
// T = float (fp32 arithmetic) or __nv_bfloat16 (tcgen05 kernel, fp32 accumulation).
template <typename T>
void FcForward(const TinyTensor<T>& input, TinyTensor<T>& output, const TinyTensor<T>& weight, const TinyTensor<T>& bias);

// grad_input = grad_output . weight^T, grad_weight = input^T . grad_output, grad_bias = column sums
// of grad_output (their total for a [1] bias) -- the reference's FcBackward (src/Layers.cu:42-79),
// same argument order; `output` is accepted and ignored as there.
template <typename T>
void FcBackward(const TinyTensor<T>& input, const TinyTensor<T>& output, const TinyTensor<T>& weight,
                const TinyTensor<T>& bias, TinyTensor<T>& grad_input, const TinyTensor<T>& grad_output,
                TinyTensor<T>& grad_weight, TinyTensor<T>& grad_bias);

#endif  // TT_HOST_LAYERS_H
