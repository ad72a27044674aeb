"""Drop-in for the reference's ``packkv_cuda`` extension module: same eight callables
(packkv_cuda_ext/export_packkv.cpp:9-18), implemented by packkv_b200 on sm_100a."""
from packkv_b200.api import (fused_kq, fused_wv, k_decode_cpu, k_encode_cpu, kq_mat_vec_mul, v_decode_cpu,
                             v_encode_cpu, wv_mat_vec_mul)

__all__ = ["k_encode_cpu", "k_decode_cpu", "kq_mat_vec_mul", "v_encode_cpu", "v_decode_cpu", "wv_mat_vec_mul",
           "fused_kq", "fused_wv"]
