"""Generate the golden vectors under tests/golden/ from the reference's own Python code.

Run once in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It loads the reference's helper module `deep_gemm/utils/math.py` by file path (it
needs only torch) and evaluates, on CPU tensors and seeded inputs,
  * the helpers themselves (`ceil_to_ue8m0`, `_quantize_to_fp4_e2m1`,
    `per_token_cast_to_fp4`, `per_token_cast_to_fp8`), and
  * the pure-torch quantised MoE of `sm100_b200/test_mega_moe.py:66-98,411-499`,
    transcribed here formula by formula on top of those imported helpers (the test
    itself cannot be imported: it needs GPUs and the compiled extension).
The outputs are what `tests/test_oracle.py` pins the CPU oracle against. The
vectors, not this script, travel with the repository's test-suite.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_math(ref_root):
    path = os.path.join(ref_root, 'deep_gemm', 'utils', 'math.py')
    spec = importlib.util.spec_from_file_location('ref_math', path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def helper_vectors(rm):
    g = torch.Generator().manual_seed(1234)
    x = torch.randn((16, 256), generator=g) * torch.logspace(-3, 2, 16)[:, None]
    x[3, 5:40] = 0
    x[7] = 0
    xb = x.to(torch.bfloat16)
    out = {'x': x.numpy(), 'x_bf16_as_f32': xb.float().numpy()}
    out['ceil_to_ue8m0'] = rm.ceil_to_ue8m0(x).numpy()
    grid = torch.cat([torch.linspace(-7, 7, 1121), torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.75, -3.5])])
    out['fp4_grid'] = grid.numpy()
    out['fp4_grid_codes'] = rm._quantize_to_fp4_e2m1(grid).view(torch.uint8).numpy()
    p, sf = rm.per_token_cast_to_fp4(xb, use_ue8m0=True, gran_k=32)
    out['cast_fp4_packed'] = p.view(torch.uint8).numpy()
    out['cast_fp4_sf'] = sf.numpy()
    q, sfp = rm.per_token_cast_to_fp8(xb, use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
    out['cast_fp8_bytes'] = q.view(torch.uint8).numpy()
    out['cast_fp8_sf_packed'] = sfp.numpy()
    np.savez_compressed(os.path.join(HERE, 'quant_helpers.npz'), **out)


def moe_vectors(rm, act_format):
    """`sm100_b200/test_mega_moe.py` torch reference on 2 simulated ranks (CPU)."""
    sf_vec = {'fp8': 32, 'mxfp4': 32, 'nvfp4': 16}[act_format]
    num_ranks, num_experts, topk, hidden, inter, clamp = 2, 8, 2, 256, 128, 10.0
    e_local = num_experts // num_ranks
    tokens = [3, 2]
    FP4 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float)

    def fp4_sf_for(amax):                                   # test_mega_moe.py:68-72
        if act_format == 'nvfp4':
            return (amax / 6.0).to(torch.float8_e4m3fn).float()
        return rm.ceil_to_ue8m0(amax / 6.0)

    def cast_to_fp4_rows(t, vec, rule):                     # test_mega_moe.py:78-93
        m, k = t.shape
        g = t.float().view(m, k // vec, vec)
        amax = g.abs().amax(dim=-1).clamp_min(1e-30)
        sf = rule(amax)
        codes = rm._quantize_to_fp4_e2m1(g / sf.unsqueeze(-1)).view(m, k)
        packed = (codes[:, 0::2] & 0x0F) | ((codes[:, 1::2] & 0x0F) << 4)
        return packed.contiguous(), sf

    def dequant(packed, sf, vec):                            # test_mega_moe.py:94-98,414-419
        u = packed.view(torch.uint8)
        codes = torch.stack([(u & 0xF), (u >> 4)], dim=-1).reshape(*u.shape[:-1], u.shape[-1] * 2).long()
        return FP4[codes] * sf.repeat_interleave(vec, dim=-1)

    def requant_per32_ue8m0(a):                              # test_mega_moe.py:425-429
        g = a.view(a.shape[0], -1, 32)
        amax = g.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
        sf = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
        return ((g / sf).to(torch.float8_e4m3fn).float() * sf).view_as(a)

    def requant_fp4(a):                                      # test_mega_moe.py:430-437
        g = a.view(a.shape[0], -1, sf_vec)
        amax = g.abs().amax(dim=-1).clamp_min(1e-30)
        sf = fp4_sf_for(amax)
        codes = rm._quantize_to_fp4_e2m1(g / sf.unsqueeze(-1))
        return (FP4[codes.view(torch.uint8).long()] * sf.unsqueeze(-1)).view_as(a)

    out = {}
    xs, idxs, ws, W1, W2 = [], [], [], [], []
    for r in range(num_ranks):
        torch.manual_seed(100 + r)                           # test_mega_moe.py:40
        x = torch.randn((tokens[r], hidden)).to(torch.bfloat16)
        w1 = (torch.randn((e_local, 2 * inter, hidden)) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn((e_local, hidden, inter)) * 0.05).to(torch.bfloat16)
        scores = torch.randn((tokens[r], num_experts))
        tw, ti = torch.topk(scores, topk, dim=-1, largest=True, sorted=False)   # :111-112
        tw = torch.softmax(tw, dim=-1)
        if act_format == 'fp8':
            xq, xsf_packed = rm.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
            xsf = (xsf_packed.view(torch.uint8).to(torch.int32) << 23).view(torch.float).view(tokens[r], -1)
            x_dq = xq.float() * xsf.repeat_interleave(32, dim=-1)                # :420-424
            out[f'x_q_{r}'] = xq.view(torch.uint8).numpy()
        else:
            xq, xsf = cast_to_fp4_rows(x, sf_vec, fp4_sf_for)
            x_dq = dequant(xq, xsf, sf_vec)
            out[f'x_q_{r}'] = xq.view(torch.uint8).numpy()
        out[f'x_sf_{r}'] = xsf.numpy()
        wvec = 32 if act_format == 'fp8' else sf_vec
        wrule = (lambda a: rm.ceil_to_ue8m0(a / 6.0)) if act_format == 'fp8' else fp4_sf_for
        q1 = [cast_to_fp4_rows(w1[e], wvec, wrule) for e in range(e_local)]
        q2 = [cast_to_fp4_rows(w2[e], wvec, wrule) for e in range(e_local)]
        out[f'w1_q_{r}'] = torch.stack([a for a, _ in q1]).view(torch.uint8).numpy()
        out[f'w1_sf_{r}'] = torch.stack([b for _, b in q1]).numpy()
        out[f'w2_q_{r}'] = torch.stack([a for a, _ in q2]).view(torch.uint8).numpy()
        out[f'w2_sf_{r}'] = torch.stack([b for _, b in q2]).numpy()
        out[f'topk_idx_{r}'] = ti.numpy()
        out[f'topk_weights_{r}'] = tw.numpy()
        xs.append(x_dq); idxs.append(ti); ws.append(tw)
        W1.append(torch.stack([dequant(a, b, wvec) for a, b in q1]))
        W2.append(torch.stack([dequant(a, b, wvec) for a, b in q2]))
    X_all, IDX_all, W_all = torch.cat(xs), torch.cat(idxs), torch.cat(ws)    # :442-444
    y_part = torch.zeros((X_all.shape[0], hidden), dtype=torch.float)
    for r in range(num_ranks):
        for el in range(e_local):                                            # :451-484
            e = r * e_local + el
            t_ids, s_ids = torch.nonzero(IDX_all == e, as_tuple=True)
            if t_ids.numel() == 0:
                continue
            h = X_all[t_ids] @ W1[r][el].T
            gate, up = h[:, :inter].to(torch.bfloat16), h[:, inter:].to(torch.bfloat16)
            gate = torch.clamp_max(gate, clamp); up = torch.clamp(up, -clamp, clamp)
            gate, up = gate.float(), up.float()
            act = gate * torch.sigmoid(gate) * up * W_all[t_ids, s_ids][:, None]
            act = requant_per32_ue8m0(act) if act_format == 'fp8' else requant_fp4(act)
            y_part.index_add_(0, t_ids, act @ W2[r][el].T)
    out['y_ref'] = y_part.numpy()
    out['tokens'] = np.array(tokens)
    out['meta'] = np.array([num_ranks, num_experts, topk, hidden, inter])
    np.savez_compressed(os.path.join(HERE, f'moe_small_{act_format}.npz'), **out)


if __name__ == '__main__':
    if len(sys.argv) != 2:
        sys.exit('usage: python tests/golden/make_golden.py <path of the reference checkout>')
    ref_root = sys.argv[1]
    rm = load_reference_math(ref_root)
    helper_vectors(rm)
    for fmt in ('mxfp4', 'nvfp4', 'fp8'):
        moe_vectors(rm, fmt)
    print('golden vectors written to', HERE)
