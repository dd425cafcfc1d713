from .sparse_index_flash_attn import (  # noqa: F401
    dense_index_flash_attn_func,
    sparse_index_flash_attn_bhtd_func,
    sparse_index_flash_attn_func,
    sparse_index_flash_attn_inference_bhtd_func,
    sparse_index_flash_attn_inference_func,
    sparse_index_flash_attn_value_gate_bhtd_func,
)
