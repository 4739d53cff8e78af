"""Stand-in for the third-party package ``torch-einops-utils`` (pinned by the reference as
``>=0.0.14``), which is not installed where the golden vectors are generated.

The reference uses exactly one helper from it, once (PoPE_pytorch/pope.py:14,64): select the
trailing ``length`` entries of ``t`` along ``dim``.  That contract is fixed inside the
reference by its decode-shape tests (tests/test_pope.py:26-29) and by the fused kernels'
``q_offset = seq_k - seq_q`` (PoPE_pytorch/triton_pope_flash_attn.py:54).  It performs no
arithmetic.  Used only by make_golden.py.
"""


def slice_right_at_dim(t, length, dim=-1):
    size = t.shape[dim]
    return t.narrow(dim, size - length, length)
