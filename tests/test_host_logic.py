"""CPU-side checks: the library loads and exports the declared C ABI, the buffer layout, the weight pre-tiling."""
import ctypes
import os
import re

import pytest
import torch

import hopper_megamoe_basedondeepgemm_b200 as mm
from hopper_megamoe_basedondeepgemm_b200 import _lib, quant
from oracle import megamoe_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    header = open(os.path.join(ROOT, 'include', 'megamoe_b200.h')).read()
    declared = set(re.findall(r'\b(mm_[a-z0-9_]+)\s*\(', header))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert getattr(lib, name) is not None


def _layout(**kw):
    lib = _lib.load()
    cfg = _lib.MMConfig(kw.get('ranks', 8), kw.get('rank', 0), kw.get('experts', 384), kw.get('tmax', 128), 8,
                        kw.get('hidden', 3072), kw.get('inter', 1280), _lib.FMT[kw.get('fmt', 'mxfp4')], 148)
    L = _lib.MMLayout()
    return lib.mm_get_layout(ctypes.byref(cfg), ctypes.byref(L)), L


def test_layout_regions_are_ordered_and_sized():
    st, L = _layout()
    assert st == 0
    offs = [L.off_ctrl, L.off_x, L.off_x_sf, L.off_topk_idx, L.off_topk_weights, L.off_rx, L.off_mid,
            L.off_mid_sf, L.off_comb, L.off_red, L.off_cnt, L.off_logits, L.off_token_tiles, L.off_mid_tiles, L.off_arrive,
            L.total_bytes]
    assert offs == sorted(offs) and all(o % 1024 == 0 for o in offs)
    # tile images (launches with more than 16 received rows): one per 16 rows of the intermediate pool at most; per tile 32
    # row records of 16 B (token tiles), then per 256-element K unit a record of 32 rows x 128 B + two scale-word slot planes
    rec32 = 32 * 128 + 2 * 32 * 16
    assert L.tile_capacity == L.mid_rows // 16
    assert L.token_tile_bytes == 32 * 16 + (3072 // 256) * rec32 and L.mid_tile_bytes == (1280 // 256) * rec32
    assert L.off_mid_tiles - L.off_token_tiles >= L.tile_capacity * L.token_tile_bytes
    assert L.off_arrive - L.off_mid_tiles >= L.tile_capacity * L.mid_tile_bytes
    assert L.total_bytes - L.off_arrive >= 2 * 2 * L.tile_capacity * 4
    assert L.x_row_bytes == 1536 and L.x_sf_row_bytes == 96 and L.rx_row_bytes == 1536 + 96 + 16
    assert L.rx_cap_rows == 128 * 8 and L.mid_row_bytes == 640 and L.mid_sf_row_bytes == 48
    assert L.rx_region_bytes >= 32 + 2 * L.rx_cap_rows * L.rx_row_bytes
    assert L.off_mid - L.off_rx >= 2 * 8 * L.rx_region_bytes
    st, L2 = _layout(fmt='nvfp4')
    assert st == 0 and L2.x_sf_row_bytes == 192 and L2.mid_sf_row_bytes == 80 and L2.sf_vec == 16


def test_layout_rejects_bad_shapes():
    assert _layout(hidden=3000)[0] == 2        # unsupported
    assert _layout(experts=385)[0] == 1        # invalid: not divisible by ranks
    assert _layout(ranks=16, experts=384)[0] == 1
    assert _layout(ranks=1, experts=384)[0] == 2   # more than 64 local experts
    assert _layout(fmt='fp8')[0] in (0, 2)


@pytest.mark.parametrize('fmt', ['mxfp4', 'nvfp4'])
def test_pretiled_stream_decodes_back_to_the_weights(fmt):
    """Walk the stream with the address arithmetic the kernel uses and recover every weight byte and scale byte."""
    vec = quant.SF_VEC[fmt]
    torch.manual_seed(0)
    e, n, k = 2, 256, 512
    w = (torch.randn(e, n, k) * 0.05).to(torch.bfloat16)
    q, sf_mn = quant.cast_grouped_weights_to_fp4(w, fmt)
    stream = quant.pretile_weights(q, sf_mn, vec)
    planes = 256 // (4 * vec)
    assert stream.shape == (e, n // 128, k // 256, 16384 + planes * 512)
    qb = q.view(torch.uint8)
    sfb = sf_mn.contiguous().view(torch.uint8).reshape(e, n, k // vec)
    for ex in range(e):
        for j in range(n // 128):
            for u in range(k // 256):
                unit = stream[ex, j, u]
                for r in (0, 1, 7, 8, 37, 64, 127):
                    for ci in range(8):
                        off = (r >> 3) * 1024 + (r & 7) * 128 + ((ci ^ (r & 7)) << 4)
                        assert torch.equal(unit[off:off + 16], qb[ex, 128 * j + r, u * 128 + ci * 16:u * 128 + ci * 16 + 16])
                    for pl in range(planes):
                        off = 16384 + pl * 512 + ((r & 31) * 4 + (r >> 5)) * 4
                        g = u * planes + pl
                        assert torch.equal(unit[off:off + 4], sfb[ex, 128 * j + r, 4 * g:4 * g + 4])


def test_product_quantiser_matches_oracle():
    torch.manual_seed(1)
    t = (torch.randn(8, 512) * 0.3).to(torch.bfloat16)
    for fmt in ('mxfp4', 'nvfp4'):
        p, sf, words = quant.cast_rows_to_fp4(t, fmt)
        po, sfo, sfbo = O.quant_fp4_rows(t, fmt, rounding='rne', sf_rule='div')
        assert torch.equal(p.view(torch.uint8), po) and torch.equal(sf, sfo)
        assert torch.equal(words.view(torch.uint8).reshape(8, -1), sfbo)


def test_interleave_matches_reference_rule():
    t = torch.arange(2 * 32).reshape(2, 32, 1)
    out = quant.interleave_gate_up(t)
    # [gate 0..7, up 0..7, gate 8..15, up 8..15]
    assert out[0, :, 0].tolist() == list(range(0, 8)) + list(range(16, 24)) + list(range(8, 16)) + list(range(24, 32))


def test_transform_weights_shapes():
    torch.manual_seed(2)
    w1 = (torch.randn(2, 512, 512) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(2, 512, 256) * 0.05).to(torch.bfloat16)
    l1, l2 = mm.transform_weights_for_mega_moe(quant.cast_grouped_weights_to_fp4(w1, 'mxfp4'),
                                               quant.cast_grouped_weights_to_fp4(w2, 'mxfp4'))
    assert l1[0].shape == (2, 4, 2, 17408) and l1[1].tolist() == [512, 512, 32]
    assert l2[0].shape == (2, 4, 1, 17408) and l2[1].tolist() == [512, 256, 32]


def test_ctypes_mirror_matches_the_header(tmp_path):
    """Compile a C program against include/megamoe_b200.h and compare every struct's size and field offsets with the
    ctypes mirror the Python binding uses."""
    import shutil
    import subprocess
    if shutil.which('gcc') is None:
        pytest.skip('no C compiler')
    structs = {'mm_config_t': _lib.MMConfig, 'mm_layout_t': _lib.MMLayout, 'mm_weight_geometry_t': _lib.MMWeightGeometry,
               'mm_launch_args_t': _lib.MMLaunchArgs, 'mm_frontend_args_t': _lib.MMFrontendArgs,
               'mm_static_args_t': _lib.MMStaticArgs}
    header = re.sub(r'/\*.*?\*/', '', open(os.path.join(ROOT, 'include', 'megamoe_b200.h')).read(), flags=re.S)
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "megamoe_b200.h"', 'int main(void) {']
    fields = {}
    for cname, ct in structs.items():
        body = re.search(r'typedef struct \w+ \{([^}]*)\} ' + cname + ';', header).group(1)
        names = []
        for decl in body.split(';'):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(','):
                names.append(re.findall(r'[A-Za-z_][A-Za-z0-9_]*', part)[-1])
        fields[cname] = names
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for f in names:
            lines.append(f'printf("{cname}.{f} %zu\\n", offsetof({cname}, {f}));')
    lines += ['return 0;', '}']
    src = tmp_path / 'abi.c'
    src.write_text('\n'.join(lines))
    exe = tmp_path / 'abi'
    subprocess.run(['gcc', '-I', os.path.join(ROOT, 'include'), '-o', str(exe), str(src)], check=True)
    out = dict(line.split() for line in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.splitlines())
    for cname, ct in structs.items():
        assert int(out[cname]) == ctypes.sizeof(ct), cname
        mirror = [f[0] for f in ct._fields_]
        assert mirror == fields[cname], (cname, mirror, fields[cname])
        for f in mirror:
            assert int(out[f'{cname}.{f}']) == getattr(ct, f).offset, (cname, f)


def test_frontend_rejects_fewer_experts_than_routes():
    """Eight routes per token cannot be drawn from fewer than eight experts: refused on the host, before any launch."""
    lib = _lib.load()
    cfg = _lib.MMConfig(1, 0, 4, 16, 8, 512, 256, _lib.FMT['mxfp4'], 148)
    dummy = ctypes.c_void_p(0x1000)                                  # never dereferenced: the argument check fails first
    fe = _lib.MMFrontendArgs(dummy, dummy, None, 4, 0, dummy, 1.0)
    assert lib.mm_frontend_launch(ctypes.byref(cfg), dummy, ctypes.byref(fe), None) == 1
    peers = (ctypes.c_void_p * 1)(0x1000)
    la = _lib.MMLaunchArgs(dummy, peers, dummy, dummy, dummy, 4, 0, None, -1.0, 1, 1.0, 1.0, 1.0, 1.0, 0.0, None)
    assert lib.mm_mega_moe_from_hidden_launch(ctypes.byref(cfg), ctypes.byref(la), ctypes.byref(fe), None) == 1


def test_tuning_values_round_trip():
    lib = _lib.load()
    old = lib.mm_get_tuning(_lib.TUNE['stages'])
    assert lib.mm_set_tuning(_lib.TUNE['stages'], 6) == 0 and lib.mm_get_tuning(_lib.TUNE['stages']) == 6
    assert lib.mm_set_tuning(_lib.TUNE['stages'], old) == 0
    assert lib.mm_set_tuning(99, 1) == 1 and lib.mm_set_tuning(0, -1) == 1 and lib.mm_get_tuning(99) == -1


@pytest.mark.parametrize('tw,vec', [(16, 32), (32, 32), (32, 16)])
def test_tile_image_reader_inverts_the_documented_layout(tw, vec):
    """Tile images (launches with more than 16 received rows): per 256-element K unit a record of `tw` rows x 128 B in
    the 128 B swizzle (16 B chunk c of row r at chunk c ^ (r & 7) of the row's 128 B, rows in groups of 8 x 128 B), then
    per scale word of the unit `tw` slots of 16 B with the word in the first 4 bytes. Images written with that address
    arithmetic are read back row by row by `SymmBuffer._rows_of_tile_images`."""
    from types import SimpleNamespace
    from hopper_megamoe_basedondeepgemm_b200.mega import SymmBuffer
    torch.manual_seed(tw + vec)
    row_bytes, tiles, header = 640, 3, 512
    units, planes = row_bytes // 128, 256 // (4 * vec)
    rec = tw * 128 + planes * tw * 16
    rows = torch.randint(0, 256, (tiles * tw, row_bytes), dtype=torch.uint8)
    words = torch.randint(0, 256, (tiles * tw, units * planes, 4), dtype=torch.uint8)
    img = torch.zeros((tiles, header + units * rec), dtype=torch.uint8)
    for t in range(tiles):
        for r in range(tw):
            for ci in range(row_bytes // 16):
                off = header + (ci >> 3) * rec + (r >> 3) * 1024 + (r & 7) * 128 + (((ci & 7) ^ (r & 7)) << 4)
                img[t, off:off + 16] = rows[t * tw + r, ci * 16:ci * 16 + 16]
            for g in range(units * planes):
                off = header + (g // planes) * rec + tw * 128 + (g % planes) * tw * 16 + r * 16
                img[t, off:off + 4] = words[t * tw + r, g]
    fake = SimpleNamespace(layout=SimpleNamespace(sf_vec=vec))
    got_rows, got_words = SymmBuffer._rows_of_tile_images(fake, img, row_bytes, tw, header)
    assert torch.equal(got_rows, rows) and torch.equal(got_words, words)


def _closed_form_schedule(nt, k, g):
    """The kernel's per-SM task list of one phase (`build_schedule` in csrc/mm_kernel.cuh), restated: NT weight-tile
    tasks of k units on G SMs. The first r = NT mod G tiles are split along K: tile t of them is shared by the SMs
    [ceil(t G / r), ceil((t + 1) G / r)), each taking one contiguous unit range (sizes differ by at most one); SM b
    then runs the whole tiles r + b, r + b + G, ... Returns per SM a list of (tile, first unit, end unit, parts)."""
    r = nt % g
    out = []
    for b in range(g):
        tasks = []
        if r:
            t = b * r // g
            gs, ge = -(-t * g // r), -(-(t + 1) * g // r)
            s, li = ge - gs, b - gs
            base, extra = k // s, k % s
            ub = li * base + min(li, extra)
            ue = ub + base + (1 if li < extra else 0)
            if ue > ub:
                tasks.append((t, ub, ue, min(s, k)))
        tasks += [(t, 0, k, 1) for t in range(r + b, nt, g)]
        out.append(tasks)
    return out


@pytest.mark.parametrize('g', [148, 132, 8])
def test_closed_form_schedule_covers_every_unit_once(g):
    """Every (tile, unit) of a phase is owned by exactly one SM, the parts of a split tile are contiguous ranges that
    agree on their count, and the SMs' unit totals differ by at most one tile's units (the arithmetic the kernel's
    scheduler runs per SM, for 16- and 32-row token tiles alike: only the number of tiles changes)."""
    for n_tiles, k in ((20, 12), (24, 5), (3, 7)):
        for m in list(range(1, 20)) + [48, 96, 113]:
            nt = m * n_tiles
            sched = _closed_form_schedule(nt, k, g)
            owner = {}
            parts = {}
            for b, tasks in enumerate(sched):
                assert sum(1 for t in tasks if t[3] > 1) <= 1          # at most one partial task per SM and phase
                for (t, ub, ue, np_) in tasks:
                    assert 0 <= ub < ue <= k
                    parts.setdefault(t, set()).add(np_)
                    for u in range(ub, ue):
                        assert (t, u) not in owner, (m, t, u)
                        owner[(t, u)] = b
            assert len(owner) == nt * k
            assert all(len(v) == 1 for v in parts.values())
            for t, v in parts.items():
                assert sum(1 for tasks in sched for x in tasks if x[0] == t) == next(iter(v))
            loads = [sum(ue - ub for (_, ub, ue, _) in tasks) for tasks in sched]
            assert max(loads) - min(loads) <= k


def test_global_scale_helper_refuses_host_tensors():
    """`nvfp4_global_scale` runs the library's reduction kernel: there is no CPU path, a host tensor is an error."""
    import hopper_megamoe_basedondeepgemm_b200 as mm
    with pytest.raises(RuntimeError):
        mm.nvfp4_global_scale(torch.ones(8))
    lib = _lib.load()
    assert lib.mm_tensor_absmax(None, 1, 8, None, None) == 1        # invalid argument: null pointers
