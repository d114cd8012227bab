"""crispybits_kernels for B200 (sm_100a): the packed W2/W3/W4 linear path of CrispyBits behind the
reference's own Python API (Crispybits/Kernel/crispybits_kernels/__init__.py exports the same names)."""
from .ops import (PackedLinearWeight, PackedLinear, packed_linear, fused_gate_up, fused_qkv,
                  candidate_split_k, balanced_split_k, virtual_rows, sm_count, max_rho, tile_n,
                  apply_rope_reference, permute_for_rope, new_workspace, set_backend, backend_name)
from .autotune import tune_gemv, tune_qkv, tune_gate_up, tune_model, TuneResult, TuneReport
from .io import from_packed_dict
from .integration import install_bitmap, load_tuning, save_tuning, FusedQKV, FusedLlamaMLP

__version__ = "0.3.0+b200"
