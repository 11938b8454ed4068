"""Helpers shared by the GPU parity tests: numpy bit patterns <-> torch device tensors, error metrics."""
import numpy as np
import torch


def dev_bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).cuda()


def dev_f16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.float16).cuda()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(t):
    """16-bit float tensor -> numpy uint16 bit patterns"""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def max_rel(a, b):
    """max |a-b| / max |b| : the tensor-scale relative error used for the attention tolerances"""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def sum_rel(a, b):
    """sum|a-b| / sum(|b|+1e-6): the metric of the reference's own parity test"""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.sum(np.abs(a - b)) / np.sum(np.abs(b) + 1e-6))


def frob_rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bf16_ulp_diff(a_bits, b_bits):
    """distance in bf16 units-in-the-last-place between two bit-pattern arrays (same-sign values)"""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + (x & 0x7FFF))
    return np.abs(key(np.asarray(a_bits)) - key(np.asarray(b_bits)))
