"""Host-side mirror of the reference's mega-MoE operator surface (`sm100_b200/mega___init__.py`).

Same names, argument meaning and error behaviour (RuntimeError on a failed check); the work is done by the
sm_100a library behind the C ABI of `include/megamoe_b200.h`. PyTorch supplies device memory, the current stream and
the symmetric-memory rendezvous only.
"""
import ctypes
from types import SimpleNamespace
from typing import Optional, Tuple

import torch

from . import _lib
from .quant import SF_VEC, interleave_gate_up, pretile_weights


def _align(x: int, y: int) -> int:
    return (x + y - 1) // y * y


def get_token_alignment_for_mega_moe() -> int:
    return int(_lib.load().mm_get_token_alignment())


class SymmBuffer:
    """The per-rank symmetric buffer and its input views (`sm100_b200/mega___init__.py:16-60`).

    `group` may be None or a one-rank group for a single GPU; then the buffer is plain device memory.
    """

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                 hidden: int, intermediate_hidden: int, use_fp8_dispatch: bool = True,
                 activation: str = 'swiglu', act_format: str = 'fp8', num_sms: int = 0, window: str = 'symm_mem'):
        assert act_format in ('fp8', 'mxfp4', 'nvfp4') and window in ('symm_mem', 'ipc')
        if activation != 'swiglu':
            raise RuntimeError('only the swiglu activation is supported')
        lib = _lib.load()
        self.act_format = act_format
        self.act_sf_vec_size = {'fp8': 0, 'mxfp4': 32, 'nvfp4': 16}[act_format]
        self.group = group
        self.num_ranks = 1 if group is None else group.size()
        self.rank = 0 if group is None else group.rank()
        self.num_experts = num_experts
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_topk = num_topk
        self.hidden = hidden
        self.intermediate_hidden = intermediate_hidden
        self.cfg = _lib.MMConfig(self.num_ranks, self.rank, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                                 intermediate_hidden, _lib.FMT[act_format], num_sms)
        self.layout = _lib.MMLayout()
        _lib.check(lib.mm_get_layout(ctypes.byref(self.cfg), ctypes.byref(self.layout)), 'get_symm_buffer_for_mega_moe')
        nbytes = int(self.layout.total_bytes)
        self._ipc = None
        if self.num_ranks > 1 and window == 'ipc':
            # the library's own window: device memory + inter-process handles, exchanged once over the group (NCCL)
            import torch.distributed as dist
            own = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(_lib.WINDOW_HANDLE_BYTES)
            _lib.check(lib.mm_window_alloc(nbytes, ctypes.byref(own), handle), 'mm_window_alloc')
            mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).cuda()
            gathered = [torch.empty_like(mine) for _ in range(self.num_ranks)]
            dist.all_gather(gathered, mine, group=group)
            blob = b''.join(bytes(t.cpu().tolist()) for t in gathered)
            peers = (ctypes.c_void_p * self.num_ranks)()
            _lib.check(lib.mm_window_open(blob, self.num_ranks, self.rank, own, peers), 'mm_window_open')
            self._ipc = (own, peers)
            self.buffer_ptrs = [int(p) for p in peers]
            self.buffer = _tensor_from_ptr(int(own.value), nbytes)
            self.handle = SimpleNamespace(buffer_ptrs=list(self.buffer_ptrs), rank=self.rank, world_size=self.num_ranks)
        elif self.num_ranks > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buffer = symm_mem.empty(nbytes, dtype=torch.int8, device='cuda')
            self.handle = symm_mem.rendezvous(self.buffer, group=group)
            self.buffer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        else:
            # one rank: plain device memory; `handle.buffer_ptrs` exists all the same (the reference's callers read it)
            self.buffer = torch.empty(nbytes, dtype=torch.int8, device='cuda')
            self.buffer_ptrs = [self.buffer.data_ptr()]
            self.handle = SimpleNamespace(buffer_ptrs=list(self.buffer_ptrs), rank=0, world_size=1)
        self.buffer.zero_()
        if self.num_ranks > 1:
            self.group.barrier()
        torch.cuda.synchronize()
        self._peer_array = (ctypes.c_void_p * self.num_ranks)(*self.buffer_ptrs)
        L, t = self.layout, num_max_tokens_per_rank
        vec = int(L.sf_vec)

        def view(off, nbytes_, dtype, shape):
            return self.buffer[off:off + nbytes_].view(dtype).view(*shape)
        # packed E2M1 pairs as int8 [t, hidden / 2], or E4M3 [t, hidden] for the FP8-activation variant
        self.x = view(L.off_x, t * L.x_row_bytes, torch.float8_e4m3fn if act_format == 'fp8' else torch.int8,
                      (t, int(L.x_row_bytes)))
        self.x_sf = view(L.off_x_sf, t * L.x_sf_row_bytes, torch.int32, (t, hidden // (4 * vec)))
        self.topk_idx = view(L.off_topk_idx, t * num_topk * 8, torch.int64, (t, num_topk))
        self.topk_weights = view(L.off_topk_weights, t * num_topk * 4, torch.float32, (t, num_topk))
        # the four input views are neighbours in the buffer: one copy of this region moves them all (see host_inputs)
        self.inputs = self.buffer[int(L.off_x):int(L.off_rx)]
        # receive pool: [parity][source rank][32 B header line, then rows of (tokens | scale bytes | 16 B record)];
        # every 8 bytes hold 4 data bytes and the launch's flag word
        self.l1_acts = view(L.off_rx, 2 * self.num_ranks * L.rx_region_bytes, torch.uint8,
                            (2, self.num_ranks, int(L.rx_region_bytes)))
        # intermediate pool (flagged words too): rows of 2 * mid_row_bytes, and per (row, L1 tile of 64 columns) one
        # word {scale bytes, launch flag}; `l2_acts_payload()` / `l2_acts_sf_payload()` strip the flags
        self.l2_acts = view(L.off_mid, L.mid_rows * 2 * L.mid_row_bytes, torch.uint8,
                            (int(L.mid_rows), 2 * int(L.mid_row_bytes)))
        self.l2_acts_sf = view(L.off_mid_sf, L.mid_rows * (intermediate_hidden // 64) * 8, torch.uint8,
                               (int(L.mid_rows), (intermediate_hidden // 64) * 8))
        # launches with more than 16 received rows keep the same rows as ready-made operand tiles instead (per 16-row
        # tile: K atoms of 16 rows x 128 B in the tensor core's swizzled order, then one 16 B slot per (scale word, row))
        self.token_tiles = view(L.off_token_tiles, L.tile_capacity * L.token_tile_bytes, torch.uint8,
                                (int(L.tile_capacity), int(L.token_tile_bytes)))
        self.mid_tiles = view(L.off_mid_tiles, L.tile_capacity * L.mid_tile_bytes, torch.uint8,
                              (int(L.tile_capacity), int(L.mid_tile_bytes)))
        # expert outputs coming back: per (token, slot) hidden / 2 flagged words {2 bf16, launch flag}
        self.combine = view(L.off_comb, t * num_topk * hidden * 4, torch.int32, (t, num_topk, hidden // 2, 2))

    def host_inputs(self):
        """A pinned host mirror of the input region and typed views into it (`x`, `x_sf`, `topk_idx`, `topk_weights`,
        shaped like the device views). Fill the views, then `sym_buffer.inputs.copy_(mirror, non_blocking=True)` moves
        all inputs of a step with a single host-to-device copy."""
        L, t = self.layout, self.num_max_tokens_per_rank
        mirror = torch.zeros(int(L.off_rx - L.off_x), dtype=torch.int8).pin_memory()
        base = int(L.off_x)

        def view(off, nbytes_, like):
            return mirror[off - base:off - base + nbytes_].view(like.dtype).view(*like.shape)
        views = {'x': view(int(L.off_x), t * int(L.x_row_bytes), self.x),
                 'x_sf': view(int(L.off_x_sf), t * int(L.x_sf_row_bytes), self.x_sf),
                 'topk_idx': view(int(L.off_topk_idx), t * self.num_topk * 8, self.topk_idx),
                 'topk_weights': view(int(L.off_topk_weights), t * self.num_topk * 4, self.topk_weights)}
        return mirror, views

    def tile_image_rows(self) -> int:
        """Rows per token tile (16 or 32) if the latest launch kept its received and intermediate rows as tile images
        (more than 16 received rows), 0 if it kept them as flagged rows. Synchronises the stream."""
        return int(self.device_status()[1][2])

    def _rows_of_tile_images(self, tiles: torch.Tensor, row_bytes: int, tw: int, header: int):
        """(rows uint8 [tiles * tw, row_bytes], scale words uint8 [tiles * tw, words, 4]) of tile images: per K unit a
        record of tw rows x 128 B (128 B swizzle) followed by the unit's scale-word slots (16 B per (word, row))."""
        planes = 256 // (4 * int(self.layout.sf_vec))
        rec, units = tw * 128 + planes * tw * 16, row_bytes // 128
        tiles = tiles.cpu()[:, header:header + units * rec]
        nt = tiles.size(0)
        recs = tiles.reshape(nt, units, rec)
        tok = recs[:, :, :tw * 128].reshape(nt, units, tw, 8, 16)                # [tile][unit][row][stored chunk][16 B]
        r = torch.arange(tw).view(tw, 1)
        stored = (torch.arange(8).view(1, 8) ^ (r & 7)).view(1, 1, tw, 8, 1).expand(nt, units, tw, 8, 16)
        rows = torch.gather(tok, 3, stored).permute(0, 2, 1, 3, 4).reshape(nt * tw, row_bytes)
        slots = recs[:, :, tw * 128:].reshape(nt, units, planes, tw, 16)         # [tile][unit][plane][row][16 B slot]
        words = slots[..., :4].permute(0, 3, 1, 2, 4).reshape(nt * tw, units * planes, 4)
        return rows.contiguous(), words.contiguous()

    def l2_acts_payload(self) -> torch.Tensor:
        """The intermediate rows of the latest launch without flag words or swizzle: uint8 [mid_rows, mid_row_bytes]."""
        tw = self.tile_image_rows()
        if tw:
            return self._rows_of_tile_images(self.mid_tiles, int(self.layout.mid_row_bytes), tw, 0)[0]
        rows = self.l2_acts.size(0)
        return self.l2_acts.view(torch.int32).view(rows, -1, 2)[..., 0].contiguous().view(torch.uint8).view(rows, -1)

    def l2_acts_sf_payload(self) -> torch.Tensor:
        """The intermediate rows' scale bytes, K-major: uint8 [mid_rows, intermediate / vec]."""
        tw = self.tile_image_rows()
        if tw:
            words = self._rows_of_tile_images(self.mid_tiles, int(self.layout.mid_row_bytes), tw, 0)[1]
            return words.reshape(words.size(0), -1)[:, :self.intermediate_hidden // int(self.layout.sf_vec)].contiguous()
        rows = self.l2_acts_sf.size(0)
        words = self.l2_acts_sf.view(torch.int32).view(rows, -1, 2)[..., 0].contiguous().view(torch.uint8).view(rows, -1, 4)
        per_tile = 64 // int(self.layout.sf_vec)
        return words[..., :per_tile].contiguous().view(rows, -1)

    def received_records(self):
        """The routed rows this rank received in its latest launch, as the kernel recorded them in the receive pool:
        per source rank a list of (local expert, token, slot, top-k weight) in arrival (= row) order. The canonical
        slot map follows from it: the rows of an expert, by (source rank, token, slot). Synchronises the stream."""
        st, words = self.device_status()
        launches = int(words[1])
        if launches == 0:
            return [[] for _ in range(self.num_ranks)]
        flag, parity = launches, (launches - 1) & 1
        L = self.layout
        row2, out = 2 * int(L.rx_row_bytes), []
        pool = self.l1_acts[parity].cpu()
        for src in range(self.num_ranks):
            region = pool[src]
            head = region[:32].view(torch.int32)
            if int(head[1]) != flag:
                out.append(None)                       # that source's header line never arrived in this launch
                continue
            recs = []
            for i in range(int(head[0])):
                w = region[32 + i * row2 + row2 - 32:32 + (i + 1) * row2].view(torch.int32)
                if any(int(w[k]) != flag for k in (1, 3, 5, 7)):
                    recs.append(None)
                    continue
                recs.append((int(w[0]) & 0xFF, int(w[2]), int(w[4]), float(w[6:7].view(torch.float32))))
            out.append(recs)
        return out

    def reset(self):
        """Zero the control block and the flags (after an aborted launch). All ranks call it together."""
        lib = _lib.load()
        torch.cuda.synchronize()
        if self.num_ranks > 1:
            self.group.barrier()
        _lib.check(lib.mm_reset(ctypes.byref(self.cfg), self.buffer.data_ptr(),
                                torch.cuda.current_stream().cuda_stream), 'reset')
        torch.cuda.synchronize()
        if self.num_ranks > 1:
            self.group.barrier()

    def device_status(self):
        """(status code, 16 status words) of the launches so far; synchronises the current stream."""
        lib = _lib.load()
        words = (ctypes.c_uint32 * 16)()
        st = lib.mm_read_device_status(ctypes.byref(self.cfg), self.buffer.data_ptr(), words,
                                       torch.cuda.current_stream().cuda_stream)
        return st, list(words)

    def phase_stamps(self):
        lib = _lib.load()
        stamps = (ctypes.c_uint64 * 32)()
        _lib.check(lib.mm_read_phase_stamps(ctypes.byref(self.cfg), self.buffer.data_ptr(), stamps,
                                            torch.cuda.current_stream().cuda_stream), 'phase_stamps')
        return list(stamps)

    def sm_phases(self):
        """Per-SM phase times of the last launch: tensor int64 [256, 32] (globaltimer ns, 0 = not reached); the slot
        meanings are listed beside `mm_read_sm_phases` in the header. Synchronises the stream."""
        lib = _lib.load()
        out = (ctypes.c_uint64 * (256 * 32))()
        _lib.check(lib.mm_read_sm_phases(ctypes.byref(self.cfg), self.buffer.data_ptr(), out,
                                         torch.cuda.current_stream().cuda_stream), 'sm_phases')
        return torch.tensor(list(out), dtype=torch.int64).view(256, 32)

    def destroy(self):
        if self._ipc is not None:
            torch.cuda.synchronize()
            own, peers = self._ipc
            self.buffer = self.x = self.x_sf = self.topk_idx = self.topk_weights = self.inputs = None
            self.l1_acts = self.l2_acts = self.l2_acts_sf = self.combine = self.token_tiles = self.mid_tiles = None
            if self.group is not None:
                self.group.barrier()                     # nobody unmaps a buffer a peer's kernel may still write
            _lib.load().mm_window_close(peers, self.num_ranks, self.rank, own)
            self._ipc = None
        self.handle = None
        self.buffer = None
        self.group = None
        self.x = None
        self.x_sf = None


def _tensor_from_ptr(ptr: int, nbytes: int) -> torch.Tensor:
    """An int8 CUDA tensor over memory this process did not allocate through torch (the library's own window)."""
    class _Mem:
        __cuda_array_interface__ = {'shape': (nbytes,), 'typestr': '|i1', 'data': (ptr, False), 'version': 3}
    return torch.as_tensor(_Mem(), device='cuda')


def get_symm_buffer_for_mega_moe(group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                                 hidden: int, intermediate_hidden: int, use_fp8_dispatch: bool = True,
                                 activation: str = 'swiglu', act_format: str = 'fp8', num_sms: int = 0,
                                 window: str = 'symm_mem') -> SymmBuffer:
    """`sm100_b200/mega___init__.py:63-78`: the token count is rounded up to the operator's alignment."""
    num_max_tokens_per_rank = _align(num_max_tokens_per_rank, get_token_alignment_for_mega_moe())
    return SymmBuffer(group, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                      use_fp8_dispatch, activation, act_format, num_sms, window)


def nvfp4_global_scale(t: torch.Tensor) -> float:
    """Per-tensor NVFP4 global scale of a CUDA bf16 / fp32 tensor: largest magnitude / (6 * 448), so that the largest
    per-16 block scale is the largest E4M3 value. The reduction is the library's `mm_tensor_absmax` kernel; the
    result comes back to the host (load time / calibration, not the hot path)."""
    if not t.is_cuda or t.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError('nvfp4_global_scale takes a CUDA bf16 or fp32 tensor')
    if t.numel() == 0:
        return 0.0
    t = t.contiguous()
    if t.data_ptr() % 16:
        t = t.clone()                                     # (a view that starts inside a 16 B word: the kernel loads 16 B at a time)
    out = torch.zeros(1, dtype=torch.float32, device=t.device)
    _lib.check(_lib.load().mm_tensor_absmax(t.data_ptr(), 1 if t.dtype == torch.bfloat16 else 0, t.numel(), out.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream), 'nvfp4_global_scale')
    return float(out.item()) / (6.0 * 448.0)


def transform_weights_for_mega_moe(l1_weights: Tuple[torch.Tensor, torch.Tensor],
                                   l2_weights: Tuple[torch.Tensor, torch.Tensor]):
    """Load-time weight transform (`sm100_b200/mega___init__.py:102-111`).

    Inputs as the reference takes them: `(packed int8 [E, N, K/2], scales int32 [E, N, K/(4 vec)] MN-major)`; fp32
    scales `[E, N, K/vec]` (what `transform_sf_into_required_layout` accepts, `csrc/apis/layout.hpp:14-60`) are taken
    too and turned into scale bytes on the way. L1 gets the 8-row gate/up interleave; both layers are pre-tiled into
    the stream the kernel copies verbatim, by one CUDA copy kernel (`mm_transform_weights`; `quant.pretile_weights`
    is its torch restatement, used for host tensors and as the test's reference). Each result is `(stream uint8 [E, N/128, K/256, unit_bytes], shape int64 [N, K, vec])`.
    """
    def one(wt, interleave):
        w, sf = wt
        e, n, kh = w.shape
        if sf.dtype == torch.float32:                  # one fp32 scale per block: [E, N, K / vec]
            vec = (kh * 2) // sf.shape[-1]
        else:                                          # int32 words of four scale bytes: [E, N, K / (4 vec)]
            vec = (kh * 2) // (sf.shape[-1] * 4)
        if vec not in (16, 32):
            raise RuntimeError('weight scale tensor must hold one scale per 16 or 32 elements')
        shape = torch.tensor([n, kh * 2, vec], dtype=torch.int64)
        if not w.is_cuda:                              # host tensors (layout tests): the torch restatement of the kernel
            if sf.dtype == torch.float32:
                raise RuntimeError('fp32 weight scales are converted by the CUDA transform: move the tensors to the GPU')
            if interleave:
                w, sf = interleave_gate_up(w), interleave_gate_up(sf)
            return pretile_weights(w, sf, vec), shape
        lib = _lib.load()
        geo = _lib.MMWeightGeometry()
        lib.mm_get_weight_geometry(_lib.FMT['nvfp4' if vec == 16 else 'mxfp4'], ctypes.byref(geo))
        w = w.contiguous()
        out = torch.empty((e, n // 128, (kh * 2) // 256, int(geo.unit_bytes)), dtype=torch.uint8, device=w.device)
        _lib.check(lib.mm_transform_weights(w.data_ptr(), sf.data_ptr(), int(sf.dtype == torch.float32), sf.stride(0),
                                            sf.stride(1), sf.stride(2), e, n, kh * 2, vec, int(interleave), out.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream), 'transform_weights_for_mega_moe')
        return out, shape
    return one(l1_weights, True), one(l2_weights, False)


def _input_region_ptr(sym_buffer: 'SymmBuffer', host_inputs):
    """Address of a pinned host mirror of the buffer's input region (from `SymmBuffer.host_inputs()`), or None."""
    if host_inputs is None:
        return None
    L = sym_buffer.layout
    if (host_inputs.device.type != 'cpu' or not host_inputs.is_pinned() or not host_inputs.is_contiguous()
            or host_inputs.numel() * host_inputs.element_size() != int(L.off_rx - L.off_x)):
        raise RuntimeError('host_inputs must be the pinned mirror returned by SymmBuffer.host_inputs()')
    return host_inputs.data_ptr()


def _launch(y, l1_weights, l2_weights, sym_buffer: SymmBuffer, stats, recipe, activation, activation_clamp, fast_math,
            engine='umma', global_scales=(1.0, 1.0, 1.0, 1.0), timeout_ms=0.0, host_inputs=None):
    lib = _lib.load(check=(engine == 'check'))          # the cross-check engine lives in the test build of the library
    if activation != 'swiglu':
        raise RuntimeError('only the swiglu activation is supported')
    b = sym_buffer
    vec = b.act_sf_vec_size or 32        # FP8 tokens carry one UE8M0 scale per 32 elements, like the MXFP4 weights
    if tuple(recipe) != (1, 1, vec):
        raise RuntimeError(f'recipe {recipe} does not match the buffer format {b.act_format}')
    if y.dtype != torch.bfloat16 or y.dim() != 2 or y.size(1) != b.hidden or not y.is_contiguous() or \
            not (y.is_cuda or y.is_pinned()):
        raise RuntimeError('y must be a contiguous bf16 [num_tokens, hidden] tensor')
    if y.size(0) > b.num_max_tokens_per_rank:
        raise RuntimeError('more tokens than the buffer was created for')
    e_local = b.num_experts // b.num_ranks
    (w1, s1), (w2, s2) = l1_weights, l2_weights
    if w1.dtype != torch.uint8 or w1.dim() != 4 or w2.dtype != torch.uint8 or w2.dim() != 4:
        raise RuntimeError('weights must come from transform_weights_for_mega_moe')
    if s1.tolist() != [2 * b.intermediate_hidden, b.hidden, vec] or s2.tolist() != [b.hidden, b.intermediate_hidden, vec]:
        raise RuntimeError('weight shapes do not match the buffer')
    if w1.size(0) != e_local or w2.size(0) != e_local or not (w1.is_contiguous() and w2.is_contiguous()):
        raise RuntimeError('expected one contiguous weight stream per local expert')
    if stats is not None and (stats.dtype != torch.int32 or stats.numel() != e_local):
        raise RuntimeError('cumulative_local_expert_recv_stats must be int32 [num_local_experts]')
    args = _lib.MMLaunchArgs(
        b.buffer.data_ptr(), b._peer_array, w1.data_ptr(), w2.data_ptr(), y.data_ptr() if y.numel() else None,
        y.size(0), _lib.ENGINE[engine], stats.data_ptr() if stats is not None else None,
        float(activation_clamp) if activation_clamp is not None else -1.0, int(bool(fast_math)),
        *[float(g) for g in global_scales], float(timeout_ms), _input_region_ptr(b, host_inputs))
    _lib.check(lib.mm_mega_moe_launch(ctypes.byref(b.cfg), ctypes.byref(args), torch.cuda.current_stream().cuda_stream),
               'mega_moe launch')


def fp4_fp4_mega_moe(y: torch.Tensor, l1_weights, l2_weights, sym_buffer: SymmBuffer,
                     cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                     recipe: Optional[Tuple[int, int, int]] = None, activation: str = 'swiglu',
                     activation_clamp: Optional[float] = None, fast_math: bool = True, *,
                     x_global_scale: float = 1.0, l1_global_scale: float = 1.0, l2_global_scale: float = 1.0,
                     mid_global_scale: float = 1.0, engine: str = 'umma', timeout_ms: float = 0.0,
                     host_inputs: Optional[torch.Tensor] = None):
    """W4A4 MegaMoE, packed E2M1 activations and weights (`sm100_b200/mega___init__.py:244-274`).

    The caller has written `x`, `x_sf`, `topk_idx`, `topk_weights[:y.size(0)]` into the buffer views; the launch is
    asynchronous on the current CUDA stream and every rank of the group must make the same call. The keyword-only
    arguments are additions: NVFP4 per-tensor scales (default 1.0 = the reference's behaviour), `engine='check'`
    (the same kernel with CUDA-core dot products, used as an on-device cross-check), the device wait budget, and
    `host_inputs`: the pinned mirror of `SymmBuffer.host_inputs()`; when given, the kernel reads this call's inputs
    straight from that host memory (no host-to-device copy is needed before the launch; `y` may likewise be a pinned
    host tensor).
    """
    assert sym_buffer.act_format in ('mxfp4', 'nvfp4'), 'buffer must be created with act_format mxfp4/nvfp4'
    if recipe is None:
        recipe = (1, 1, sym_buffer.act_sf_vec_size)
    assert recipe[2] == sym_buffer.act_sf_vec_size
    _launch(y, l1_weights, l2_weights, sym_buffer, cumulative_local_expert_recv_stats, recipe, activation,
            activation_clamp, fast_math, engine, (x_global_scale, l1_global_scale, l2_global_scale, mid_global_scale),
            timeout_ms, host_inputs)


def fp8_fp4_mega_moe(y: torch.Tensor, l1_weights, l2_weights, sym_buffer: SymmBuffer,
                     cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                     recipe: Tuple[int, int, int] = (1, 1, 32), activation: str = 'swiglu',
                     activation_clamp: Optional[float] = None, fast_math: bool = True, *,
                     engine: str = 'umma', timeout_ms: float = 0.0, host_inputs: Optional[torch.Tensor] = None):
    """W-MXFP4 x A-FP8 MegaMoE (`sm100_b200/mega___init__.py:221-241`).

    Tokens are E4M3 with one UE8M0 scale per 32 elements, the intermediate is requantised the same way, weights are
    the MXFP4 streams of `transform_weights_for_mega_moe`. The tensor cores read 4-bit operands of an 8-bit x 4-bit
    product from byte-wide slots, so the kernel widens each streamed weight unit in shared memory; HBM traffic is
    that of the W4A4 variant.
    """
    assert sym_buffer.act_format == 'fp8', 'buffer must be created with act_format fp8'
    _launch(y, l1_weights, l2_weights, sym_buffer, cumulative_local_expert_recv_stats, recipe, activation,
            activation_clamp, fast_math, engine, (1.0, 1.0, 1.0, 1.0), timeout_ms, host_inputs)


def mega_moe_from_hidden(y: torch.Tensor, hidden: torch.Tensor, router_weight: torch.Tensor, l1_weights, l2_weights,
                         sym_buffer: SymmBuffer, workspace: torch.Tensor,
                         cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                         activation_clamp: Optional[float] = None, fast_math: bool = True, score_mode: int = 0,
                         expert_bias: Optional[torch.Tensor] = None, x_global_scale: float = 1.0,
                         l1_global_scale: float = 1.0, l2_global_scale: float = 1.0, mid_global_scale: float = 1.0,
                         engine: str = 'umma', timeout_ms: float = 0.0):
    """The whole layer from bf16 hidden states in ONE persistent kernel: router GEMM, top-8, routing weights and token
    quantisation run at the head of the launch, then dispatch, both grouped GEMMs and the combine. The reference runs
    its frontend as a separate kernel in the same CUDA graph (`sm100_b200/fe_sm100/test_e2e_b200.py:204-231`). The
    routing and the quantised tokens still land in `sym_buffer.topk_idx / topk_weights / x / x_sf`."""
    lib = _lib.load()
    b = sym_buffer
    if hidden.dtype != torch.bfloat16 or router_weight.dtype != torch.bfloat16 or not hidden.is_contiguous():
        raise RuntimeError('hidden states and router weight must be contiguous bf16')
    if hidden.size(0) != y.size(0) or hidden.size(1) != b.hidden or tuple(router_weight.shape) != (b.num_experts, b.hidden):
        raise RuntimeError('router shapes do not match the buffer')
    if workspace.numel() * workspace.element_size() < fe_workspace_bytes(b):
        raise RuntimeError('frontend workspace too small')
    (w1, _), (w2, _) = l1_weights, l2_weights
    stats = cumulative_local_expert_recv_stats
    args = _lib.MMLaunchArgs(
        b.buffer.data_ptr(), b._peer_array, w1.data_ptr(), w2.data_ptr(), y.data_ptr() if y.numel() else None,
        y.size(0), _lib.ENGINE[engine], stats.data_ptr() if stats is not None else None,
        float(activation_clamp) if activation_clamp is not None else -1.0, int(bool(fast_math)),
        float(x_global_scale), float(l1_global_scale), float(l2_global_scale), float(mid_global_scale),
        float(timeout_ms), None)
    fe = _lib.MMFrontendArgs(hidden.data_ptr(), router_weight.data_ptr(),
                             expert_bias.data_ptr() if expert_bias is not None else None,
                             hidden.size(0), score_mode, workspace.data_ptr(), float(x_global_scale))
    _lib.check(lib.mm_mega_moe_from_hidden_launch(ctypes.byref(b.cfg), ctypes.byref(args), ctypes.byref(fe),
                                                  torch.cuda.current_stream().cuda_stream), 'mega_moe_from_hidden')


def set_tuning(**kwargs) -> None:
    """Development knobs of the kernel (`mm_set_tuning`): knobs=<bit mask>, stages=<ring depth>,
    prefetch_w1_experts=<n>, prefetch_w2_experts=<n>. Process-wide; every rank must use the same values."""
    lib = _lib.load()
    for k, v in kwargs.items():
        _lib.check(lib.mm_set_tuning(_lib.TUNE[k], int(v)), f'set_tuning({k})')


def fe_workspace_bytes(e) -> int:
    """`fe_workspace_bytes(e)` of `sm100_b200/fe_sm100/fe_binding.cpp:30`; a `SymmBuffer` is accepted in place of the
    expert count (then the size covers the buffer's token capacity)."""
    lib = _lib.load()
    if isinstance(e, SymmBuffer):
        return max(int(lib.mm_frontend_workspace_bytes(ctypes.byref(e.cfg))), int(lib.mm_fe_workspace_bytes(e.num_experts)))
    return int(lib.mm_fe_workspace_bytes(int(e)))


def fe_router_ctas(m: int, h: int, e: int, topk: int) -> int:
    """`fe_router_ctas(m, h, e, topk)` of `sm100_b200/fe_sm100/fe_binding.cpp:31`."""
    return int(_lib.load().mm_fe_router_ctas(int(m), int(h), int(e), int(topk)))


def fe_forward(hidden: torch.Tensor, router_weight: torch.Tensor, x: torch.Tensor, x_sf: torch.Tensor,
               topk_idx: torch.Tensor, topk_weights: torch.Tensor, workspace: torch.Tensor, mode: int, l2_persist: int = 1):
    """Router frontend with the reference's argument list (`sm100_b200/fe_sm100/fe_binding.cpp:8-28`): router GEMM,
    top-8 + softmax over the selected logits, and the token quantisation (mode 2 FP8 / 3 MXFP4 / 4 NVFP4), written into
    the given views (normally `sym_buffer.x / x_sf / topk_idx / topk_weights`). The checks are the reference's."""
    lib = _lib.load()
    if hidden.dim() != 2 or hidden.dtype != torch.bfloat16 or not hidden.is_contiguous():
        raise RuntimeError('hidden must be a contiguous bf16 [m, h] tensor')
    if router_weight.dim() != 2 or router_weight.dtype != torch.bfloat16 or not router_weight.is_contiguous():
        raise RuntimeError('router_weight must be a contiguous bf16 [e, h] tensor')
    m, h = hidden.shape
    e, topk = router_weight.size(0), topk_idx.size(1)
    if router_weight.size(1) != h or not (1 <= m <= 64):
        raise RuntimeError('router shapes do not match (1 <= m <= 64)')
    if topk_idx.dtype != torch.int64 or topk_weights.dtype != torch.float32:
        raise RuntimeError('topk_idx must be int64 and topk_weights float32')
    if topk_idx.size(0) < m or topk_weights.size(0) < m or x.size(0) < m or x_sf.size(0) < m:
        raise RuntimeError('output views hold fewer than m rows')
    row = h if mode == 2 else h // 2
    sf_row = h // (16 if mode == 4 else 32)
    if x.stride(0) * x.element_size() != row or x_sf.stride(0) * x_sf.element_size() != sf_row or \
            not (topk_idx[:m].is_contiguous() and topk_weights[:m].is_contiguous()):
        raise RuntimeError('output views do not have the row strides of the activation format')
    nbytes = workspace.numel() * workspace.element_size()
    _lib.check(lib.mm_fe_forward(hidden.data_ptr(), router_weight.data_ptr(), x.data_ptr(), x_sf.data_ptr(),
                                 topk_idx.data_ptr(), topk_weights.data_ptr(), workspace.data_ptr(), nbytes, m, h, e, topk,
                                 int(mode), int(l2_persist), torch.cuda.current_stream().cuda_stream), 'fe_forward')


def fe_forward_into_buffer(hidden: torch.Tensor, router_weight: torch.Tensor, sym_buffer: SymmBuffer, workspace: torch.Tensor,
                           score_mode: int = 0, expert_bias: Optional[torch.Tensor] = None, x_global_scale: float = 1.0):
    """The frontend with this build's extensions (sigmoid + bias scores, NVFP4 global scale, any token count up to the
    buffer's capacity), written into `sym_buffer.x / x_sf / topk_idx / topk_weights[:hidden.size(0)]`."""
    lib = _lib.load()
    b = sym_buffer
    if hidden.dtype != torch.bfloat16 or router_weight.dtype != torch.bfloat16:
        raise RuntimeError('hidden states and router weight must be bf16')
    if hidden.size(1) != b.hidden or tuple(router_weight.shape) != (b.num_experts, b.hidden):
        raise RuntimeError('router shapes do not match the buffer')
    if workspace.numel() * workspace.element_size() < fe_workspace_bytes(b):
        raise RuntimeError('frontend workspace too small')
    args = _lib.MMFrontendArgs(hidden.data_ptr(), router_weight.data_ptr(),
                               expert_bias.data_ptr() if expert_bias is not None else None,
                               hidden.size(0), score_mode, workspace.data_ptr(), float(x_global_scale))
    _lib.check(lib.mm_frontend_launch(ctypes.byref(b.cfg), b.buffer.data_ptr(), ctypes.byref(args),
                                      torch.cuda.current_stream().cuda_stream), 'fe_forward_into_buffer')
