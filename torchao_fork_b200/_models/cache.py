"""Per-sequence memory of the models: key/value caches of the gpt-fast Llama (plain and int8), and the state of
sequence models that keep something else per request — compressed (latent) keys, the previous token's input of a
token-shift layer, a ring of keys and values for attention that never looks past a fixed span (with a small store beside it for
first tokens that stay visible for good), the state of a
recurrence (a vector or a matrix per head), the last inputs of a short convolution — in numbered slots that a host-side allocator hands out and takes
back.
"""
from typing import Dict, List, Optional

import torch
import torch.nn as nn


class KVCache(nn.Module):
    """reference: model.py:166-192.  [B][n_local_heads][S][head_dim]"""

    def __init__(self, max_batch_size, max_seq_length, n_heads, head_dim, dtype=torch.bfloat16):
        super().__init__()
        shape = (max_batch_size, n_heads, max_seq_length, head_dim)
        self.register_buffer("k_cache", torch.zeros(shape, dtype=dtype))
        self.register_buffer("v_cache", torch.zeros(shape, dtype=dtype))

    def update(self, input_pos, k_val, v_val):
        assert input_pos.shape[0] == k_val.shape[2]
        self.k_cache[:, :, input_pos] = k_val
        self.v_cache[:, :, input_pos] = v_val
        return self.k_cache, self.v_cache


class AffineQuantizedKVCache(nn.Module):
    """reference: model.py:198-240.  int8 rows [B][n_local_heads][S][head_dim] + one scale per row
    [B][n_local_heads][S][1]; update() returns the dequantized caches with the positions just written replaced by the
    unquantized values.  (Decode steps do not call update(): csrc/decode_attn_q8.cu does the same thing for the new
    row inside the attention launch and never materialises the dequantized cache.)"""

    def __init__(self, max_batch_size, max_seq_length, n_heads, head_dim, scale_dtype=torch.bfloat16):
        super().__init__()
        cache_shape = (max_batch_size, n_heads, max_seq_length, head_dim)
        scale_shape = (max_batch_size, n_heads, max_seq_length, 1)
        self.register_buffer("k_cache", torch.zeros(cache_shape, dtype=torch.int8))
        self.register_buffer("v_cache", torch.zeros(cache_shape, dtype=torch.int8))
        self.register_buffer("k_cache_scale", torch.ones(scale_shape, dtype=scale_dtype))
        self.register_buffer("v_cache_scale", torch.ones(scale_shape, dtype=scale_dtype))

    def update(self, input_pos, k_val, v_val):
        from ..quantization.utils import _quantize_activation_per_token_absmax
        q_k_val, k_scale = _quantize_activation_per_token_absmax(k_val)
        self.k_cache[:, :, input_pos] = q_k_val
        self.k_cache_scale[:, :, input_pos] = k_scale.unsqueeze(-1)
        k_out = self.k_cache * self.k_cache_scale
        k_out[:, :, input_pos] = k_val
        q_v_val, v_scale = _quantize_activation_per_token_absmax(v_val)
        self.v_cache[:, :, input_pos] = q_v_val
        self.v_cache_scale[:, :, input_pos] = v_scale.unsqueeze(-1)
        v_out = self.v_cache * self.v_cache_scale
        v_out[:, :, input_pos] = v_val
        return k_out, v_out

    @classmethod
    def from_float(cls, kv_cache):
        max_batch_size, n_heads, max_seq_length, head_dim = kv_cache.k_cache.shape
        return cls(max_batch_size, max_seq_length, n_heads, head_dim, kv_cache.k_cache.dtype)


class SlotAllocator:
    """Hands out the slot numbers 0 .. n-1 of a slotted cache.  A freed slot is handed out again (lowest number first,
    so that reuse is exercised early); whatever its rows hold is overwritten by the next owner position by position and
    never read beyond the owner's own length."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots))

    def alloc(self) -> int:
        if not self._free:
            raise RuntimeError(f"all {self.n_slots} sequence slots are in use")
        self._free.sort()
        return self._free.pop(0)

    def free(self, slot: int) -> None:
        assert 0 <= slot < self.n_slots and slot not in self._free, slot
        self._free.append(slot)

    def grow(self, n_slots: int) -> None:
        assert n_slots >= self.n_slots
        self._free += list(range(self.n_slots, n_slots))
        self.n_slots = n_slots

    @property
    def in_use(self) -> int:
        return self.n_slots - len(self._free)


class LatentKVCache(nn.Module):
    """What a latent-attention layer keeps per position instead of keys and values: the normed latent
    `c` [slots][S][rank] and the rotated key part shared by all heads `kr` [slots][S][rot_dim]."""

    def __init__(self, n_slots, max_seq_length, rank, rot_dim, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.register_buffer("c", torch.zeros(n_slots, max_seq_length, rank, dtype=dtype, device=device))
        assert rank > 0 and rot_dim > 0
        self.register_buffer("kr", torch.zeros(n_slots, max_seq_length, rot_dim, dtype=dtype, device=device))

    def grow(self, n_slots):
        for name in ("c", "kr"):
            old = getattr(self, name)
            new = torch.zeros(n_slots, *old.shape[1:], dtype=old.dtype, device=old.device)
            new[: old.shape[0]] = old
            setattr(self, name, new)


class TokenShiftState(nn.Module):
    """The input row of a sequence's last token, per slot, in fp32: the next step's first token mixes with it."""

    def __init__(self, n_slots, width, device=None):
        super().__init__()
        self.register_buffer("prev", torch.zeros(n_slots, width, dtype=torch.float32, device=device))

    def grow(self, n_slots):
        new = torch.zeros(n_slots, self.prev.shape[1], dtype=torch.float32, device=self.prev.device)
        new[: self.prev.shape[0]] = self.prev
        self.prev = new


def _grown(old: torch.Tensor, n_slots: int) -> torch.Tensor:
    new = torch.zeros(n_slots, *old.shape[1:], dtype=old.dtype, device=old.device)
    new[: old.shape[0]] = old
    return new


class RingKVCache(nn.Module):
    """Keys and values of an attention that only ever reads the last `ring` positions or less (a chunked or a sliding
    mask): position p of a sequence lives in row p % ring of its slot, k [slots][ring][kv_heads][dim] and
    v [slots][ring][kv_heads][vdim].  What a sequence costs does not grow with its length."""

    def __init__(self, n_slots, ring, kv_heads, dim, vdim, dtype=torch.bfloat16, device=None):
        super().__init__()
        assert ring > 0
        self.ring = ring
        self.register_buffer("k", torch.zeros(n_slots, ring, kv_heads, dim, dtype=dtype, device=device))
        self.register_buffer("v", torch.zeros(n_slots, ring, kv_heads, vdim, dtype=dtype, device=device))

    def grow(self, n_slots):
        self.k, self.v = _grown(self.k, n_slots), _grown(self.v, n_slots)


class WindowKVCache(nn.Module):
    """Keys and values of an attention whose mask is a sliding window plus the first tokens of the sequence: a ring of
    `ring` rows (>= the widest window of the layers that read it; position p in row p % ring) and, beside it, the first
    `first_rows` positions (>= the most first tokens that any reader keeps), which the ring's turning never reaches.
    k_width / v_width are whole rows (all key/value heads, all attention maps of a head).  What a sequence costs does not
    grow with its length."""

    def __init__(self, n_slots, ring, first_rows, k_width, v_width, dtype=torch.bfloat16, device=None):
        super().__init__()
        assert ring > 0 and first_rows >= 0
        self.ring, self.first_rows = ring, first_rows
        self.register_buffer("k", torch.zeros(n_slots, ring, k_width, dtype=dtype, device=device))
        self.register_buffer("v", torch.zeros(n_slots, ring, v_width, dtype=dtype, device=device))
        self.register_buffer("k_first", torch.zeros(n_slots, max(1, first_rows), k_width, dtype=dtype, device=device))
        self.register_buffer("v_first", torch.zeros(n_slots, max(1, first_rows), v_width, dtype=dtype, device=device))

    def grow(self, n_slots):
        self.k, self.v = _grown(self.k, n_slots), _grown(self.v, n_slots)
        self.k_first, self.v_first = _grown(self.k_first, n_slots), _grown(self.v_first, n_slots)


class RecurrentState(nn.Module):
    """The state of a per-channel recurrence, fp32 [slots][width]; a sequence starts from zeros (the kernels do not
    read the slot at position 0, so a reused slot needs no clearing)."""

    def __init__(self, n_slots, width, device=None):
        super().__init__()
        self.register_buffer("s", torch.zeros(n_slots, width, dtype=torch.float32, device=device))

    def grow(self, n_slots):
        self.s = _grown(self.s, n_slots)


class MatrixState(nn.Module):
    """The state of a recurrence that keeps a matrix per head (decayed linear attention, state-space duality): fp32
    [slots][heads][rows][cols]; a sequence starts from zeros (the kernel does not read the slot at position 0, so a reused
    slot needs no clearing)."""

    def __init__(self, n_slots, heads, rows, cols, device=None):
        super().__init__()
        self.register_buffer("s", torch.zeros(n_slots, heads, rows, cols, dtype=torch.float32, device=device))

    def grow(self, n_slots):
        self.s = _grown(self.s, n_slots)


class ConvState(nn.Module):
    """The last taps - 1 inputs of a causal convolution over time, fp32 [slots][taps - 1][channels], oldest first (a
    one-tap convolution remembers nothing: it keeps one unused row so that the buffer exists)."""

    def __init__(self, n_slots, taps, channels, device=None):
        super().__init__()
        assert taps >= 1
        self.taps = taps
        self.register_buffer("x", torch.zeros(n_slots, max(1, taps - 1), channels, dtype=torch.float32, device=device))

    def grow(self, n_slots):
        self.x = _grown(self.x, n_slots)


class SequenceStates:
    """State manager of a slotted model: which request owns which slot and how many positions it has written.  The
    device buffers themselves belong to the model's layers (LatentKVCache, TokenShiftState); `on_grow` callbacks
    enlarge them when more requests are alive than slots exist."""

    def __init__(self, n_slots: int, max_seq_length: int):
        self.alloc = SlotAllocator(n_slots)
        self.max_seq_length = max_seq_length
        self.length: Dict[int, int] = {}       # slot -> positions written
        self.owner: Dict[object, int] = {}     # request id -> slot
        self.on_grow = []

    def slot_of(self, request) -> int:
        """The request's slot; a new request gets a free one (doubling the slot count if none is left)."""
        if request not in self.owner:
            if self.alloc.in_use == self.alloc.n_slots:
                n = 2 * self.alloc.n_slots
                for cb in self.on_grow:
                    cb(n)
                self.alloc.grow(n)
            s = self.alloc.alloc()
            self.owner[request] = s
            self.length[s] = 0
        return self.owner[request]

    def extend(self, slot: int, n_tokens: int) -> int:
        """Reserves the next n_tokens positions of the slot's sequence; returns the first of them."""
        at = self.length[slot]
        if at + n_tokens > self.max_seq_length:
            raise RuntimeError(f"sequence of {at + n_tokens} tokens does not fit the cache ({self.max_seq_length} positions per slot)")
        self.length[slot] = at + n_tokens
        return at

    def release(self, request) -> None:
        s = self.owner.pop(request)
        del self.length[s]
        self.alloc.free(s)

    def reset(self) -> None:
        for r in list(self.owner):
            self.release(r)
