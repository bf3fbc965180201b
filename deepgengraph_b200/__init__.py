"""deepgengraph_b200 -- B200 (sm_100a) implementation of the fused attention core modules of
FlashTensor / DeepGenGraph and of its csrc/ bandwidth ops, behind the reference's operator API.

  native_ops   rms_norm / silu_and_mul / rotary_embedding_online (+ fused_add_rms_norm,
               gelu_tanh_and_mul): same names and argument order as the reference's csrc/ffi.cpp
  attention    attn_fwd / attn_score_fwd / attn_kf_fwd on BSHD tensors (also torch custom ops)
  kernels      KERNEL_ZOO-compatible modules (Attn, Gemma2, H2O, RoCo, KeyFormer) with prepare()
  compile      compile(model, input_names, inputs, output_names, system='b200') -> f
  sharding     batch x head partitioning over the GPUs of one node
  layer        Gemma-2-style decoder layer glue built on the ops above

Everything computes on the GPU through libb200attn.so; there is no CPU or eager fallback.
"""
__version__ = "0.1.0"
