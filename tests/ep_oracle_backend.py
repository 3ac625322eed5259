"""CPU stand-in for the CUDA kernels used by croqtile_b200.moe_ep: the same
operations computed by the oracle on torch CPU tensors. Lets the exchange logic
run as gloo ranks without a GPU. Test infrastructure only."""
import numpy as np
import torch

from oracle import oracle as o


def _bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _from_bf16_bits(b):
    return torch.from_numpy(np.ascontiguousarray(b).view(np.int16)).view(torch.bfloat16)


def _e4m3(t):
    return t.contiguous().view(torch.uint8).numpy()


def _to_e4m3(b):
    return torch.from_numpy(np.ascontiguousarray(b)).view(torch.float8_e4m3fn)


class OracleBackend:
    def route(self, logits, k):
        r = o.moe_route_topk(logits.numpy(), k)
        return {key: torch.from_numpy(v) for key, v in r.items()}

    def permute_quant(self, x, perm_to_src, k):
        rows = o.bf16_to_f32(_bf16_bits(x))[perm_to_src.numpy() // k]
        q, s = o.quant_rows_e4m3(rows)
        return _to_e4m3(q), torch.from_numpy(s)

    def quant_rows(self, x):
        q, s = o.quant_rows_e4m3(o.bf16_to_f32(_bf16_bits(x)))
        return _to_e4m3(q), torch.from_numpy(s)

    def grouped_gemm(self, x, xs, w, ws, offsets, swiglu):
        out = o.moe_grouped_gemm_e4m3(_e4m3(x), xs.numpy(), _e4m3(w), ws.numpy(), offsets.numpy(), swiglu)
        return _from_bf16_bits(out)

    def gather_rows(self, src, index):
        return src[index.long()].contiguous()

    def unpermute(self, y, src_to_perm, topk_w):
        return _from_bf16_bits(o.moe_unpermute(_bf16_bits(y), src_to_perm.numpy(), topk_w.numpy()))
