"""bf16 GEMM front end for the tcgen05 kernel (``csrc/gemm_sm100.cu``).

``gemm(a, b)`` contracts over K with either operand stored K-major (``[rows, K]``) or MN-major
(``[K, rows]``), which covers forward (``x @ W.T``), input-gradient (``dy @ W``) and
weight-gradient (``dy.T @ x``) products without materialising a transpose. The epilogue flags
fuse bias, GELU (keeping the pre-activation), GELU', residual add, SiLU, element-wise and
per-row scaling, fp32 output and accumulation into the destination.

On CPU tensors the same contract is evaluated with plain torch in fp32 (used by the CPU tests);
on CUDA tensors only the native kernel runs.
"""
from __future__ import annotations

import os

import torch

from .. import _C

EPI_BIAS = 1
EPI_GELU = 2
EPI_DGELU = 4
EPI_ADD_AUX = 8
EPI_OUT_F32 = 16
EPI_ACCUMULATE = 32
EPI_SILU = 64
EPI_MUL_AUX = 128
EPI_SCATTER_PEERS = 256
EPI_ROW_SCALE = 512
TALL = 1 << 12   # or-ed into the tile width: 256-row tiles (two 128-row MMAs per B stage)
PAIR = 1 << 13   # or-ed into the tile width: CTA-pair kernel (cta_group::2), 256 x 256 tiles over two SMs
_PAIR = {"mode": os.environ.get("MOMIJO_GEMM_PAIR", "auto")}   # "0" never, "1" whenever eligible, "auto"


def _gelu_tanh(x):
    return torch.nn.functional.gelu(x, approximate="tanh")


def _gelu_tanh_grad(x):
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def pick_bn(M: int, N: int) -> int:
    """N tile width: 256 keeps the MMA at its widest; narrower tiles for narrow outputs."""
    if N <= 64:
        return 64
    if N <= 128:
        return 128
    sms = 148
    best, best_cost = 256, None
    for bn in (256, 128):
        tiles = -(-M // 128) * -(-N // bn)
        waves = -(-tiles // sms)
        cost = waves * bn * (1.0 if bn == 256 else 1.12)  # narrow tiles re-read A more often
        if best_cost is None or cost < best_cost:
            best, best_cost = bn, cost
    return best


_SPLITK = {"ranges": {}, "scratch": None, "enabled": True, "force": None}


# Measured cost of one 64-deep K block of a tile, in SM cycles (B200, operands streamed from L2/HBM):
# the taller / wider the tile, the fewer operand bytes it pulls per FLOP.
_KBLOCK_CYCLES = {(128, False): 850.0, (256, False): 1100.0, (128, True): 1230.0, (256, True): 2100.0}
_PAIR_KBLOCK_CYCLES = 920.0   # 256 x 256 tile on a CTA pair (128 x 256 per SM, half of B staged per SM)


def plan_wgrad(M: int, N: int, K: int):
    """(splits, tile width, tall) for a weight-gradient shaped product dW[M, N] = sum_k dy[k, M] x[k, N]
    (small output, long contraction). The output alone has too few tiles to occupy 148 SMs, so the
    contraction is cut into S ranges whose partial products run as separate tiles (fp32 slabs) and are
    summed by one reduction pass. Returns S = 1 when the plain kernel is the better choice."""
    if _SPLITK["force"] is not None:
        f = _SPLITK["force"]
        return f if isinstance(f, tuple) else (max(1, int(f)), 128, False)
    plain_tiles = -(-M // 128) * -(-N // 128)
    if not _SPLITK["enabled"] or K < 4096 or plain_tiles >= 2 * 148:
        return 1, 128, False
    best, best_cost = (1, 128, False), None
    cands = list(_KBLOCK_CYCLES.items())
    if _PAIR["mode"] != "0" and M >= 256 and N >= 256:
        cands.append(((256, "pair"), _PAIR_KBLOCK_CYCLES))
    for (bn, tall), kcyc in cands:
        if bn > max(128, N) or (tall and M < 256):
            continue
        tiles = -(-M // (256 if tall else 128)) * -(-N // bn)
        units = 74 if tall == "pair" else 148        # a pair tile occupies two SMs
        for S in range(1, 17):
            if K // S < 1024:
                break
            waves = -(-(tiles * S) // units)
            cost = waves * (K / S / 64.0) * kcyc
            if S > 1 or tall:
                cost += 5700.0 + S * M * N * 0.0026    # reduction pass: launch + slab traffic
            if best_cost is None or cost < best_cost - 1e-6:
                best, best_cost = (S, bn, tall), cost
    S, bn, tall = best
    if S == 1 and tall:      # a single range needs no slabs: fall back to the plain kernel (which picks
        # its own tile shape, the pair kernel included)
        return 1, 128, False
    return best


def plan_split_k(M: int, N: int, K: int, bn: int = 128):
    return plan_wgrad(M, N, K)[0]


def pick_tall(M: int, N: int, K: int) -> bool:
    """256 x 256 tiles for plain products with a long contraction and enough tiles to fill the GPU
    several times over: they pull a third less operand data per FLOP than 128 x 256 tiles, at the price
    of an epilogue that no longer overlaps the next tile's main loop (which is why short contractions
    keep the 128-row tiles)."""
    return K >= 4096 and M >= 256 and N >= 256 and (-(-M // 256)) * (-(-N // 256)) >= 3 * 148


def pick_pair(M: int, N: int, K: int) -> bool:
    """CTA-pair kernel for plain products: each SM of a pair stages half of the 256-wide B tile, so a
    256 x 256 tile costs a third less L2 -> shared-memory traffic per FLOP than 128 x 256 on one SM, and
    (unlike the one-SM 256 x 256 tile) both accumulators still fit, so epilogues overlap main loops."""
    mode = _PAIR["mode"]
    if mode == "0" or M < 256 or N < 256:
        return False
    if mode == "1":
        return True
    # measured: ahead of the one-SM tiles by 1.2x on contractions up to 3072 deep (0.88-0.95 of cuBLAS);
    # long contractions with many tiles stay on the one-SM 256 x 256 tiles (pick_tall)
    return not pick_tall(M, N, K)


def _split_ranges(K: int, S: int, device):
    key = (K, S, str(device))
    r = _SPLITK["ranges"].get(key)
    if r is None:
        step = -(-K // S)
        step = (step + 127) // 128 * 128
        edges = [min(i * step, K) for i in range(S + 1)]
        r = torch.tensor([v for i in range(S) for v in (edges[i], edges[i + 1])], dtype=torch.int32, device=device)
        _SPLITK["ranges"][key] = r
    return r


def _gemm_split_k(a, b, out, accumulate, M, N, K, S, bn, tall=False):
    """a: [K, M], b: [K, N] (both MN-major). Partial products as fp32 slabs, then one reduction pass."""
    need = S * M * N
    sc = _SPLITK["scratch"]
    if sc is None or sc.numel() < need or sc.device != a.device:
        sc = torch.empty(need, dtype=torch.float32, device=a.device)
        _SPLITK["scratch"] = sc
    _C.call("mmj_gemm_bf16_grouped_k", _C.ptr(a), a.stride(0), _C.ptr(b), b.stride(0), _C.ptr(sc), N, K, M, N, S,
            _C.ptr(_split_ranges(K, S, a.device)), 1, 0,
            bn | (PAIR if tall == "pair" else TALL if tall else 0),
            _C.ptr(_C.status_tensor(a.device)),
            _C.current_stream())
    _C.call("mmj_splitk_reduce", _C.ptr(sc), M * N, S, _C.ptr(out), M * N, int(accumulate), _C.current_stream())
    return out


def _check_2d(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride, got shape {tuple(t.shape)} "
                         f"strides {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_f32=False, accumulate=False, bias=None,
         gelu=False, pre_out=None, dgelu_aux=None, add_aux=None, mul_aux=None, silu=False,
         row_scale=None, bn=None, tall=False, pair=None):
    """D[M, N] = contraction over K of A and B, followed by the fused epilogue.

    a: ``[M, K]`` (or ``[K, M]`` when ``a_mn``); b: ``[N, K]`` (or ``[K, N]`` when ``b_mn``).
    """
    _check_2d(a, "a")
    _check_2d(b, "b")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"contraction mismatch: {K} vs {Kb}")
    aux = dgelu_aux if dgelu_aux is not None else (add_aux if add_aux is not None else mul_aux)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
        accumulate = False
    else:
        out_f32 = out.dtype == torch.float32
        if out.dim() != 2 or out.shape[0] != M or out.shape[1] != N or out.stride(1) != 1:
            raise ValueError("bad out shape")
    if gelu and pre_out is None:
        pre_out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)

    if not a.is_cuda:
        A = (a.t() if a_mn else a).float()
        Bm = (b if b_mn else b.t()).float()
        v = A @ Bm
        if bias is not None:
            v = v + bias.float()
        if gelu:
            pre_out.copy_(v.to(torch.bfloat16))
            v = _gelu_tanh(v)
        if silu:
            v = torch.nn.functional.silu(v)
        if dgelu_aux is not None:
            v = v * _gelu_tanh_grad(dgelu_aux.float())
        elif mul_aux is not None:
            v = v * mul_aux.float()
        elif add_aux is not None:
            v = v + add_aux.float()
        if row_scale is not None:
            v = v * row_scale.float()[:, None]
        if accumulate:
            v = v + out.float()
        out.copy_(v.to(out.dtype))
        return (out, pre_out) if gelu else out

    epi = 0
    if bias is not None:
        epi |= EPI_BIAS
    if gelu:
        epi |= EPI_GELU
    if silu:
        epi |= EPI_SILU
    if dgelu_aux is not None:
        epi |= EPI_DGELU
    elif mul_aux is not None:
        epi |= EPI_MUL_AUX
    elif add_aux is not None:
        epi |= EPI_ADD_AUX
    if out_f32:
        epi |= EPI_OUT_F32
    if accumulate:
        epi |= EPI_ACCUMULATE
    if row_scale is not None:
        epi |= EPI_ROW_SCALE
    if aux is not None:
        _check_2d(aux, "aux")
    if N % 8 != 0 and out.stride(0) % 8 != 0:
        raise ValueError("output leading dimension must be a multiple of 8 elements")
    if (a_mn and b_mn and epi in (0, EPI_ACCUMULATE) and out.is_contiguous() and (M * N) % 8 == 0
            and M % 8 == 0 and N % 8 == 0):
        S, sbn, stall = plan_wgrad(M, N, K)
        if S > 1:
            return _gemm_split_k(a, b, out, accumulate, M, N, K, S, sbn, stall)
    if pair is None:
        pair = bn is None and not tall and pick_pair(M, N, K)
    if pair:
        bn, tall = 256 | PAIR, False
    elif bn is None:
        if not tall and pick_tall(M, N, K):
            bn, tall = 256, True
        else:
            bn = pick_bn(M, N)
    _C.call("mmj_gemm_bf16", _C.ptr(a), a.stride(0), int(a_mn), _C.ptr(b), b.stride(0), int(b_mn),
            _C.ptr(out), out.stride(0), M, N, K, epi, _C.ptr(bias), _C.ptr(aux),
            aux.stride(0) if aux is not None else 0, _C.ptr(pre_out),
            pre_out.stride(0) if pre_out is not None else 0, _C.ptr(row_scale), bn | (TALL if tall else 0),
            _C.ptr(_C.status_tensor(a.device)), _C.current_stream())
    return (out, pre_out) if gelu else out
