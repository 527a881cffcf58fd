"""B200-native (sm_100a) replacement for the fields-lm fused Field read.

Public surface:

* :func:`fused_field_read` - drop-in for the reference operator of the same name;
* :func:`fused_field_read_bf16` - the operator on a bfloat16 boundary (fp32 state);
* :func:`fused_field_read_bf16_stats` - the same plus the per-token sum of squares an RMS norm needs;
* :func:`field_read_with_state` - the operator with carried state in and out;
* :func:`field_read_step` - one recurrent step for incremental decoding;
* :class:`FieldStackDecoder` - stateful prefill -> decode for a field-only language model;
* :func:`fields_lm_b200.seqpar.sequence_parallel_field_read` - sequence-sharded forward;
* :func:`install` / :func:`uninstall` - rebind the operator inside a built model;
* :func:`linear_scan` - the reference's ``hierarchical_scan`` for real fp32 CUDA tensors
  (the softpatch mixer's call site), :func:`install_scan` to put it in place;
* :mod:`fields_lm_b200.mixer` - the fused mixer forward, prefill and single-token step on the
  reference's own mixer / block objects;
* :mod:`fields_lm_b200.build` - compiles the CUDA library.

The CUDA library is required: nothing here falls back to a CPU or PyTorch path.
"""
from .decode import FieldStackDecoder, field_read_step
from .field_read import (FieldReadFunction, field_read_with_state, fused_field_read,
                         fused_field_read_bf16, fused_field_read_bf16_stats)
from .install import install, install_scan, uninstall
from .scan import linear_scan, linear_scan_with_state

__all__ = ["FieldReadFunction", "FieldStackDecoder", "field_read_step", "field_read_with_state", "fused_field_read", "fused_field_read_bf16", "fused_field_read_bf16_stats", "install",
           "install_scan", "linear_scan", "linear_scan_with_state", "uninstall"]
