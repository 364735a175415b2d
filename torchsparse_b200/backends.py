"""Global switches, same names as torchsparse/backends.py:4-11.

``init`` is lazy about the device: importing the package must work on a machine
without a GPU (build and CPU-side tests run there)."""
import torch

benchmark = False
allow_tf32 = False
allow_fp16 = True
device_capability = 0
hash_rsv_ratio = 2  # table slots reserved per input point (>= 2)
# Exact-fp32 convolutions (allow_tf32 = False) of tensor-core shapes: three TF32 passes over the split operands
# (x_hi w_hi + x_hi w_lo + x_lo w_hi, fp32 accumulation) instead of the CUDA-core kernel; no counterpart in the
# reference, whose fp32 path runs on the CUDA cores
fp32_by_split_tf32 = True
# Kernel-map builds keyed by the ravel index of a coordinate use a table of 32-bit keys (one 8-byte slot per entry)
# whenever the key space of the level stays below 2^32, and the 64-bit layout otherwise; False always takes the
# 64-bit layout.  The maps are the same either way (the reference's *_hashmap_int32 builders make the same choice
# by name).
hash_keys_32bit = True


def init():
    global benchmark, allow_tf32, allow_fp16, device_capability, hash_rsv_ratio
    benchmark = False
    if torch.cuda.is_available():
        cap = torch.cuda.get_device_capability()
        device_capability = cap[0] * 100 + cap[1] * 10
    else:
        device_capability = 0
    # as in the reference: fp32 convolutions multiply as TF32 (fp32 accumulation) on Ampere and newer;
    # set allow_tf32 = False for exact fp32 arithmetic on the CUDA cores
    allow_tf32 = device_capability >= 800
    allow_fp16 = True
    hash_rsv_ratio = 2
