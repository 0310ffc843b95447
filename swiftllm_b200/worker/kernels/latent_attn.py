"""Latent attention over the paged latent cache (csrc/latent_attn.cu).  Cache layout [num_blocks, slots, block_size, r + dr]:
per token and caching layer ONE row [normed latent | rotated key part] shared by all heads."""
import torch

from swiftllm_b200 import _lib


def latent_kv_store(dkv: torch.Tensor, norm_weight: torch.Tensor, cache: torch.Tensor, slot: int, block_table: torch.Tensor,
                    infer_state, r: int, dr: int, rot_dims: int, eps: float, cos: torch.Tensor, sin: torch.Tensor):
    """dkv [T, r + dr] (row-strided): RMS-norm the first r columns, rotate the rest, write the tokens' cache rows."""
    assert dkv.dim() == 2 and dkv.stride(1) == 1 and dkv.shape[1] == r + dr and cache.is_contiguous() and cache.dtype == dkv.dtype
    _lib.require_device(dkv)
    T = dkv.shape[0]
    _lib.check(_lib.lib().sllm_latent_kv_store(
        dkv.data_ptr(), dkv.stride(0) if T > 1 else max(dkv.stride(0), r + dr), norm_weight.data_ptr(), _lib.ptr(cos), _lib.ptr(sin),
        infer_state.token_seq_ids.data_ptr(), infer_state.token_positions.data_ptr(), block_table.data_ptr(), block_table.shape[1],
        cache.data_ptr(), cache.shape[1], slot, cache.shape[2], T, r, dr, rot_dims, eps, _lib.dtype_tag_f32(dkv.dtype),
        _lib.stream()), "latent_kv_store")


_SM_COUNT = {}


def _num_splits(T: int, H: int, window: int, dtype) -> int:
    """Key splits for the tensor-core kernel: as many CTAs as fit at once (two per SM) when the step has few tokens (decoding),
    never a second wave; never more than the 64-key tiles a window can hold (16 when there is no window)."""
    if dtype == torch.float32:
        return 1
    dev = torch.cuda.current_device()
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    ctas = T * ((H + 15) // 16)
    want = (2 * _SM_COUNT[dev]) // ctas
    most = (window + 63) // 64 + 1 if window > 0 else 16
    return max(1, min(want, most, 32))


def latent_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, gate, cache: torch.Tensor, slot: int, block_table: torch.Tensor,
                     infer_state, out: torch.Tensor, rot_dims: int, window: int, scale: float, cos: torch.Tensor, sin: torch.Tensor):
    """q_lat [T, H, r], q_rot [T, H, dr] (un-rotated), gate [T, H] logits or None, out [T, H, r]; views with arbitrary token /
    head strides are taken as they are (the innermost stride must be 1)."""
    T, H, r = q_lat.shape
    dr = q_rot.shape[2]
    assert q_lat.stride(2) == 1 and q_rot.stride(2) == 1 and out.stride(2) == 1 and out.shape == q_lat.shape
    assert cache.shape[3] == r + dr and cache.dtype == q_lat.dtype
    assert gate is None or (gate.shape == (T, H) and gate.stride(1) == 1)
    _lib.require_device(q_lat)
    nsplit = _num_splits(T, H, window, q_lat.dtype)
    ws = torch.empty((T, H, nsplit, r + 2), dtype=torch.float32, device=q_lat.device) if nsplit > 1 else None
    _lib.check(_lib.lib().sllm_latent_attention(
        q_lat.data_ptr(), q_lat.stride(0), q_lat.stride(1), q_rot.data_ptr(), q_rot.stride(0), q_rot.stride(1),
        _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(gate), gate.stride(0) if gate is not None else 0,
        cache.data_ptr(), cache.shape[1], slot, cache.shape[2], block_table.data_ptr(), block_table.shape[1],
        infer_state.token_seq_ids.data_ptr(), infer_state.token_positions.data_ptr(),
        out.data_ptr(), out.stride(0), out.stride(1), T, H, r, dr, rot_dims, window, scale, nsplit, _lib.ptr(ws),
        _lib.dtype_tag_f32(q_lat.dtype), _lib.stream()), "latent_attention")
