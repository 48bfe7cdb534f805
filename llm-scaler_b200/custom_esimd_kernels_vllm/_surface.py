"""Schema strings of the ops the reference package registers that this build does not implement.

They are registered all the same (see _register.py), for the CUDA key, with an implementation that raises
`RuntimeError("b2q: <op> not implemented")`: callers of the reference probe the op surface with
`getattr(torch.ops.<ns>, name, None)` and must find every name, and a call has to fail with a clear message
rather than with a missing attribute.  The strings are the reference's own, character for character
(csrc/xpu/torch_extension*.cc, csrc/moe_batch/moe.sycl:2442-2459, csrc/moe_batch/moe_int4.sycl:3896-3937,
csrc/eagle/eagle.sycl:533-535).  What they cover: the dense 16-bit GEMV, stand-alone norm / RoPE / GDN kernels and
paged attention (outside the quantized-linear path), and the single-launch tiny-batch MoE decode variants.
"""

UNIMPLEMENTED = {
    "eagle_ops": [
        "gdn_eagle(Tensor! qkvz, Tensor! z_out, Tensor conv_w, Tensor? conv_b, Tensor! conv_state, Tensor accepted_tokens, Tensor ba, Tensor a_log, Tensor dt_bias, Tensor! state_in, Tensor ssm_state_idx, Tensor norm_w, int max_query_len) -> Tensor",
        "page_attn_decode(Tensor query, Tensor kv_cache, Tensor block_table, Tensor seq_lens, Tensor! out, int max_query_len, int max_seq_len, float k_scale=1.0, float v_scale=1.0) -> ()",
    ],
    "moe_ops": [
        "moe_router_forward(Tensor x, Tensor weight, Tensor scale) -> Tensor",
        "moe_up_forward(Tensor x, Tensor gate_up_weight, Tensor gate_up_scale, Tensor shared_gate_up_weight, Tensor shared_gate_up_scale, Tensor selected_experts, int top_k, int num_shared_experts) -> Tensor",
        "moe_down_forward(Tensor x, Tensor intermediates, Tensor down_weight, Tensor down_scale, Tensor shared_down_weight, Tensor shared_down_scale, Tensor shared_expert_gate_weight, Tensor routing_weights, Tensor selected_experts, int top_k, int num_shared_experts) -> Tensor",
        "moe_forward_fused(Tensor x, Tensor gate_up_weight, Tensor gate_up_scale, Tensor shared_gate_up_weight, Tensor shared_gate_up_scale, Tensor down_weight, Tensor down_scale, Tensor shared_down_weight, Tensor shared_down_scale, Tensor shared_expert_gate_weight, Tensor routing_weights, Tensor selected_experts, int top_k, int num_shared_experts) -> Tensor",
        "moe_forward_full(Tensor x, Tensor logits, Tensor gate_up_weight, Tensor gate_up_scale, Tensor shared_gate_up_weight, Tensor shared_gate_up_scale, Tensor down_weight, Tensor down_scale, Tensor shared_down_weight, Tensor shared_down_scale, Tensor shared_expert_gate_weight, int top_k, int num_shared_experts, int n_routed_experts) -> Tensor",
        "moe_forward_full_fp8_block(Tensor x, Tensor logits, Tensor(a!) output, Tensor gate_up_weight, Tensor gate_up_scale, Tensor shared_gate_up_weight, Tensor shared_gate_up_scale, Tensor down_weight, Tensor down_scale, Tensor shared_down_weight, Tensor shared_down_scale, Tensor shared_expert_gate_weight, int top_k, int num_shared_experts, int n_routed_experts) -> Tensor(a!)",
        "moe_forward_full_v2(Tensor x, Tensor logits, Tensor gate_up_weight, Tensor gate_up_scale, Tensor shared_gate_up_weight, Tensor shared_gate_up_scale, Tensor down_weight, Tensor down_scale, Tensor shared_down_weight, Tensor shared_down_scale, Tensor shared_expert_gate_weight, int top_k, int num_shared_experts, int n_routed_experts) -> Tensor",
    ],
    "moe_int4_ops": [
        "moe_forward_tiny_cutlass_nmajor_int4(Tensor x, Tensor w13_qweight_s4, Tensor w13_scales, Tensor w2_qweight_s4, Tensor w2_scales, Tensor topk_weight, Tensor topk_idx) -> Tensor",
        "moe_tiny_cutlass_nmajor_int4_up(Tensor x, Tensor w13_qweight_s4, Tensor w13_scales, Tensor topk_idx) -> Tensor",
        "moe_forward_gelu_tanh_int4_decode(Tensor x, Tensor logits, Tensor w13_qweight_s4, Tensor w13_scales, Tensor w2_qweight_s4, Tensor w2_scales, Tensor per_expert_scale, int top_k, int n_routed_experts) -> Tensor",
        "moe_tiny_cutlass_nmajor_int4_down(Tensor intermediates, Tensor w2_qweight_s4, Tensor w2_scales, Tensor topk_weight, Tensor topk_idx) -> Tensor",
        "moe_forward_tiny_cutlass_nmajor_int4_full_fp16_shared(Tensor x, Tensor w13_qweight_s4, Tensor w13_scales, Tensor w2_qweight_s4, Tensor w2_scales, Tensor topk_weight, Tensor topk_idx, Tensor shared_gate_up_weight, Tensor shared_down_weight, Tensor shared_expert_gate_weight, int num_shared_experts) -> Tensor",
        "moe_forward_tiny_cutlass_nmajor_int4_full_fp16_shared_from_logits(Tensor x, Tensor logits, Tensor w13_qweight_s4, Tensor w13_scales, Tensor w2_qweight_s4, Tensor w2_scales, Tensor shared_gate_up_weight, Tensor shared_down_weight, Tensor shared_expert_gate_weight, int top_k, int num_shared_experts, int n_routed_experts) -> Tensor",
        "moe_tiny_fp16_shared_up(Tensor x, Tensor shared_gate_up_weight, int num_shared_experts) -> Tensor",
        "moe_tiny_fp16_shared_finalize(Tensor x, Tensor shared_intermediates, Tensor routed_output, Tensor shared_down_weight, Tensor shared_expert_gate_weight, int num_shared_experts) -> Tensor",
    ],
    "custom_esimd_kernels_vllm": [
        "esimd_gemv_fp16(Tensor input, Tensor weight, Tensor output) -> Tensor",
        "esimd_gemv_fp16_gelu_mul(Tensor input, Tensor weight, Tensor output) -> Tensor",
        "esimd_qkv_split_norm_rope(Tensor qkv_state, Tensor(a!) q_out, Tensor(b!) gate_out, Tensor(c!) k_out, Tensor(d!) v_out, Tensor norm_wq, Tensor norm_wk, Tensor positions, int q_heads, int kv_heads, bool attn_output_gate, int rotary_dim, Tensor cos_sin_cache) -> ()",
        "esimd_qkv_split_norm_rope_v(Tensor qkv_state, Tensor(a!) q_out, Tensor(b!) gate_out, Tensor(c!) k_out, Tensor(d!) v_out, Tensor norm_wq, Tensor norm_wk, Tensor norm_wv, Tensor positions, int q_heads, int kv_heads, bool attn_output_gate, int rotary_dim, Tensor cos_sin_cache) -> ()",
        "esimd_rms_norm(Tensor input, Tensor output, Tensor weight, float eps) -> Tensor",
        "esimd_fused_add_rms_norm(Tensor hidden_states, Tensor residual, Tensor weight, float eps) -> Tensor",
        "esimd_fused_scaled_add_rms_norm(Tensor hidden_states, Tensor residual, Tensor weight, float eps, float scalar) -> Tensor",
        "esimd_rms_norm_gated(Tensor x, Tensor z, Tensor weight, Tensor output, float eps) -> Tensor",
        "esimd_fused_add_rms_norm_batched(Tensor hidden_states, Tensor residual, Tensor weight, float eps) -> Tensor",
        "esimd_norm_add_norm(Tensor h2_raw, Tensor h1, Tensor w1, Tensor w2, Tensor out, float eps1, float eps2) -> ()",
        "esimd_accum_norm_add_norm(Tensor routed_output, Tensor h1, Tensor w1, Tensor w2, Tensor out, int top_k, float eps1, float eps2) -> ()",
        "esimd_gdn_conv_fused(Tensor qkvz, Tensor(a!) conv_state, Tensor conv_weight, Tensor conv_bias, Tensor conv_state_indices, Tensor A_log, Tensor dt_bias, Tensor ba, Tensor(b!) ssm_state, Tensor ssm_state_indices, Tensor(c!) output, Tensor(d!) z_out, int N, int H, int HV, int K, int V, float scale) -> Tensor(c!)",
        "esimd_gdn_conv_fused_seq(Tensor qkvz, Tensor(a!) conv_state, Tensor conv_weight, Tensor conv_bias, Tensor conv_state_indices, Tensor A_log, Tensor dt_bias, Tensor ba, Tensor(b!) ssm_state, Tensor ssm_state_indices, Tensor(c!) output, Tensor(d!) z_out, int N, int H, int HV, int K, int V, float scale) -> Tensor(c!)",
        "esimd_gdn_conv_fused_seq_spec(Tensor qkvz, Tensor(a!) conv_state, Tensor conv_weight, Tensor conv_bias, Tensor spec_state_indices, Tensor A_log, Tensor dt_bias, Tensor ba, Tensor(b!) ssm_state, Tensor(c!) output, Tensor(d!) z_out, Tensor token_indx, Tensor num_accepted_tokens, int num_spec_decodes, int num_spec_tokens, int H, int HV, int K, int V, float scale) -> Tensor(c!)",
    ],
}
