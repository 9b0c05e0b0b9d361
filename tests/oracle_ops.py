"""A CPU stand-in for `accel_b200.runtime` built on the oracle: `launch(name, bindings, uniform)`
with the same kernel names, binding order and std140 uniform bytes, over CPU torch tensors.

Test infrastructure: it lets the host-side logic above the kernels (the decode step's wiring, the
tensor-parallel shard plan and its collectives) run as gloo ranks on a machine with no GPU, and it
gives the GPU decode test an oracle-side step to compare with.  The product never imports it."""
import struct

import numpy as np
import torch

import oracle as orc


def _np(t, dtype=None):
    a = t.numpy()
    if dtype is not None:
        a = a.view(dtype)
    return a


def _cache(t):
    return _np(t, np.uint16) if t.dtype == torch.float16 else _np(t)


def quantize(w: torch.Tensor):
    """DecodeModel's `quantize` hook: quant.Int4Quantize through the oracle, as CPU tensors."""
    p, s, z = orc.int4_quantize(w.contiguous().numpy())
    return (torch.from_numpy(p.view(np.int32)), torch.from_numpy(s.view(np.float16)),
            torch.from_numpy(z.view(np.float16)))


def launch(name, bindings, uniform=None, lengths=None, workspace=None):
    b = bindings
    u = uniform or b""
    if name in ("QuantMatMulInt4", "QuantMatVecInt4"):
        M, N, K, _ = struct.unpack("<IIII", u[:16])
        M = max(M, 1)
        out = orc.quant_matmul_int4(_np(b[0]).reshape(M, K), _np(b[1], np.uint32), _np(b[2], np.uint16),
                                    _np(b[3], np.uint16), M, N, K)
        b[4].view(-1)[:M * N].copy_(torch.from_numpy(out.ravel()))
    elif name in ("AttentionDecodeBatched", "AttentionDecodeBatchedF16"):
        B, qH, kvH, D, blk, mp, sc, _ = struct.unpack("<IIIIIIfI", u[:32])
        out = orc.attention_decode_batched(_np(b[0]), _cache(b[1]), _cache(b[2]), _np(b[3], np.uint32),
                                           _np(b[4], np.uint32), B, qH, kvH, D, blk, mp, sc)
        b[5].view(-1).copy_(torch.from_numpy(out))
    elif name == "RMSNorm":
        rows, width, eps, _ = struct.unpack("<IIfI", u[:16])
        out = orc.rmsnorm(_np(b[0]).reshape(rows, width), _np(b[1]), eps)
        b[2].view(-1).copy_(torch.from_numpy(out.ravel()))
    elif name == "RoPE":
        rows, width, rot, base = struct.unpack("<IIIf", u[:16])
        out = orc.rope(_np(b[1]).reshape(rows, width), _np(b[0], np.uint32), rot, base)
        b[1].view(-1).copy_(torch.from_numpy(out.ravel()))
    elif name in ("ScatterRows", "ScatterRowsF16"):
        rows, width, cap, _ = struct.unpack("<IIII", u[:16])
        orc.scatter_rows(_cache(b[0]), _np(b[1], np.uint32), _cache(b[2]), cap)
    elif name == "GatherRows":
        rows, width, cap, _ = struct.unpack("<IIII", u[:16])
        out = orc.gather_rows(_np(b[0]), _np(b[1], np.uint32), width, cap)
        b[2].view(-1).copy_(torch.from_numpy(out.ravel()))
    elif name == "SwiGLU":
        b[2].copy_(torch.from_numpy(orc.swiglu(_np(b[0]), _np(b[1]))))
    elif name == "ElemAdd":
        b[2].copy_(torch.from_numpy(orc.elem_add(_np(b[0]), _np(b[1]))))
    elif name == "SampleArgmax":
        vocab, rows, _, _ = struct.unpack("<IIII", u[:16])
        rows = b[1].numel()
        out = orc.sample_argmax(_np(b[0]).reshape(rows, vocab))
        b[1].copy_(torch.from_numpy(out.view(np.int32)))
    elif name == "ArgmaxShard":
        # this rank's columns -> (largest logit, index in the whole vocabulary) in its slot, zeros elsewhere
        width, rows, parts, rank, first = struct.unpack("<IIIII", u[:20])
        logits = _np(b[0]).reshape(rows, width)
        idx = orc.sample_argmax(logits).astype(np.int64)
        pairs = np.zeros((rows, parts, 2), np.float32)
        pairs[:, rank, 0] = logits[np.arange(rows), idx]
        pairs[:, rank, 1] = (first + idx).astype(np.float32)
        b[1].copy_(torch.from_numpy(pairs).view_as(b[1]))
    elif name == "ArgmaxMerge":
        rows, parts = struct.unpack("<II", u[:8])
        pairs = _np(b[0]).reshape(rows, parts, 2)
        out = np.zeros(rows, np.int32)
        for r in range(rows):
            v, i = pairs[r, 0]
            for s_ in range(1, parts):
                ov, oi = pairs[r, s_]
                if ov > v or (ov == v and oi < i):
                    v, i = ov, oi
            out[r] = int(i)
        b[1].copy_(torch.from_numpy(out))
    elif name == "SegmentOffsets":
        rows = struct.unpack("<I", u[:4])[0]
        b[1].copy_(torch.from_numpy(orc.segment_offsets(_np(b[0], np.uint32)[:rows]).view(np.int32)))
    elif name == "GroupedMatMulInt4":
        # the extension's definition: dequantize each expert's planes (quant.Int4Dequantize), then
        # the reference GroupedMatMul
        E, tokens, K, N = struct.unpack("<IIII", u[:16])
        per = K * N
        w = np.empty((E, K, N), np.float32)
        codes, sc, zr = _np(b[1], np.uint32), _np(b[2], np.uint16), _np(b[3], np.uint16)
        for e in range(E):
            w[e] = orc.int4_dequantize(codes[e * per // 8:(e + 1) * per // 8], sc[e * per // 128:(e + 1) * per // 128],
                                       zr[e * per // 128:(e + 1) * per // 128], per).reshape(K, N)
        out = orc.grouped_matmul(_np(b[0]).reshape(tokens, K), w, _np(b[4], np.uint32), tokens, E, K, N,
                                 out=_np(b[5]).reshape(tokens, N).copy())
        b[5].view(-1).copy_(torch.from_numpy(out.ravel()))
    elif name == "CastF32ToF16":
        b[1].view(-1).copy_(torch.from_numpy(orc.to_f16_bits(_np(b[0])).view(np.float16)))
    elif name == "DecodeStepInputs":
        B, hq, hk, blk, mp = struct.unpack("<IIIII", u[:20])
        sampled, pages = _np(b[0], np.uint32), _np(b[1], np.uint32).reshape(B, mp)
        tokens, pos_q, pos_k, slots, lengths = (x for x in b[2:7])
        for s in range(B):
            pos = int(lengths[s])
            tokens[s] = int(sampled[s])
            pos_q[s * hq:(s + 1) * hq] = pos
            pos_k[s * hk:(s + 1) * hk] = pos
            slots[s] = int(pages[s, pos // blk]) * blk + pos % blk if pos // blk < mp else -1
            lengths[s] = pos + 1
    else:
        raise NotImplementedError(name)
