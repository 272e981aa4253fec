"""Heterogeneous-rate LDLQ over many live encoder states, and the two candidate-grid reuse
schedules built on it.

Mirrors, with the same names, argument meaning and error behaviour
(``qsrt/exl3_encoder_backend.py``):

* ``ldlq_mixed_batched`` (``:1190-1478``): independent traversals whose 16-row steps are encoded
  together, with a buffer-aligned processing interval, continuation state and shared immutable
  sources (``source_indices``);
* ``ldlq_mixed_n_candidates_reuse`` (``:1481-1642``): output-axis rate candidates assembled from
  one all-K3 encode plus one encode of the union of their K2 / K4 columns;
* ``ldlq_mixed_k_candidates_prefix_reuse`` (``:1645-1830``): input-axis rate candidates that
  share the rows the backwards traversal visits first, continued as a trie of states.

Where the reference gathers tiles with ``index_select`` / ``cat`` and launches one kernel per
rate, a step here issues one ``qsrtb_ldlq_quantize_members`` launch per (rate, column set): the
kernel reads each state's source rows and compensation in place and scatters reconstruction,
error and states straight back, addressed through a small (source, owner) table.
"""

from __future__ import annotations

import torch

from . import _lib
from . import tiles as _tiles
from .tiles import K2_DEDICATED_MAX_LABEL, _stream_ptr, prepared_table, traceback_scratch


def _encoder():
    from . import encoder

    return encoder


class _Launches:
    """Device-side launch tables of one call: which states share a kernel launch at a row of
    tiles, keyed by the states' rates there."""

    def __init__(self, rate_axis: str, tile_bits: list[tuple[int, ...]], multipliers: tuple[float, ...],
                 tiles_n: int, sources: list[int], device: torch.device) -> None:
        self.rate_axis = rate_axis
        self.tile_bits = tile_bits
        self.multipliers = multipliers
        self.tiles_n = tiles_n
        self.sources = sources
        self.device = device
        self._by_signature: dict[tuple, list] = {}
        self._members: dict[tuple, torch.Tensor] = {}
        self._columns: dict[tuple, torch.Tensor] = {}

    def _row_bits(self, member: int, row_tile: int) -> tuple[int, ...] | int:
        bits = self.tile_bits[member]
        if self.rate_axis == "k":
            return bits[row_tile]
        if self.rate_axis == "n":
            return bits
        return bits[row_tile * self.tiles_n:(row_tile + 1) * self.tiles_n]

    def at(self, row_tile: int) -> list:
        """``[(bits, multiplier, members tensor, count, column tensor or None)]`` for one row of tiles."""

        rows = [self._row_bits(m, row_tile) for m in range(len(self.tile_bits))]
        signature = tuple(rows) if self.rate_axis != "n" else ()
        cached = self._by_signature.get(signature)
        if cached is not None:
            return cached
        groups: dict[tuple, list[int]] = {}
        for member, row in enumerate(rows):
            if isinstance(row, int):
                parts = [(row, None)]
            else:
                present = sorted(set(row))
                if len(present) == 1:
                    parts = [(present[0], None)]
                else:
                    parts = [(b, tuple(i for i, v in enumerate(row) if v == b)) for b in present]
            for bits, columns in parts:
                groups.setdefault((bits, self.multipliers[member], columns), []).append(member)
        launches = []
        for (bits, multiplier, columns), members in groups.items():
            key = tuple(members)
            table = self._members.get(key)
            if table is None:
                table = torch.tensor([[self.sources[m], m] for m in members], dtype=torch.int32, device=self.device)
                self._members[key] = table
            column_tensor = None
            if columns is not None:
                column_tensor = self._columns.get(columns)
                if column_tensor is None:
                    column_tensor = torch.tensor(columns, dtype=torch.int32, device=self.device)
                    self._columns[columns] = column_tensor
            launches.append((bits, multiplier, table, len(members), column_tensor))
        self._by_signature[signature] = launches
        return launches


def _quantize_members(weights, product_cache, weights_q, err, encoded_q, row_begin: int, launch, quant_args: dict):
    """One ``qsrtb_ldlq_quantize_members`` launch for the 16-row step starting at ``row_begin``."""

    enc = _encoder()
    bits, multiplier, table, count, columns = launch
    device = weights.device
    _, size_k, size_n = weights.shape
    lut, lut_pm, abs_max = prepared_table(enc._codebook_for(quant_args, bits), bits, device)
    dedicated = bits == 2 and abs_max == abs_max and 0.0 < abs_max <= K2_DEDICATED_MAX_LABEL
    variant, cost_rows = _tiles.search_variant(dedicated, quant_args)
    scratch = traceback_scratch(device, bits, cost_rows=cost_rows)
    visited = columns.numel() if columns is not None else size_n // 16
    row_bytes = row_begin * size_n * 4
    with torch.cuda.device(device), _tiles.timed_search(device, count * visited, bits):
        _lib.check(
            _lib.lib().qsrtb_ldlq_quantize_members(
                weights.data_ptr() + row_bytes, product_cache.data_ptr() + row_bytes, float(multiplier),
                table.data_ptr(), count, size_n, size_n, size_n, size_k * size_n, size_k * size_n,
                lut.data_ptr(), lut_pm.data_ptr(), bits, int(quant_args.get("tailbite_context", 128)),
                variant, weights_q.data_ptr() + row_bytes, err.data_ptr() + row_bytes,
                encoded_q.data_ptr() + (row_begin // 16) * (size_n // 16) * 256 * 2,
                (size_k // 16) * (size_n // 16) * 256,
                columns.data_ptr() if columns is not None else None, visited if columns is not None else 0,
                scratch.data_ptr(), scratch.numel(), _stream_ptr(device),
            ),
            "qsrtb_ldlq_quantize_members",
        )


def ldlq_mixed_batched(
    weights: torch.Tensor,
    Ls: torch.Tensor,
    quant_args_list: list[dict],
    pb=None,
    *,
    synchronize: bool = True,
    prepared_groupings=None,
    process_begin: int = 0,
    process_end: int | None = None,
    initial_weights_q: torch.Tensor | None = None,
    initial_encoded_q: torch.Tensor | None = None,
    initial_product_cache: torch.Tensor | None = None,
    return_product_cache: bool = False,
    source_indices: torch.Tensor | None = None,
):
    """Batch independent heterogeneous-rate LDLQ traversals (exl3_encoder_backend.py:1190-1478).

    ``weights [S, k, n]`` and ``Ls [S, k, k]`` are immutable sources; member ``b`` of
    ``quant_args_list`` encodes source ``b`` (or ``source_indices[b]``) with its own rate map,
    reconstruction, error feedback and product cache.  ``process_begin``/``process_end`` restrict
    the backwards traversal to one buffer-aligned interval of rows; a lower interval continues
    from the three state tensors an earlier call returned (they are updated in place and
    returned).  ``prepared_groupings`` is accepted for signature compatibility and ignored: the
    launch tables are built per call.
    """

    enc = _encoder()
    if weights.ndim != 3 or Ls.ndim != 3:
        raise ValueError("batched mixed LDLQ expects rank-three weights and Ls")
    source_count, size_k, size_n = weights.shape
    batch = len(quant_args_list)
    if source_count <= 0 or batch <= 0 or Ls.shape != (source_count, size_k, size_k):
        raise ValueError("batched mixed LDLQ weight/L shapes do not agree")
    if weights.dtype != torch.float or Ls.dtype != torch.float:
        raise TypeError("batched mixed LDLQ weights and Ls must be float32")
    if weights.device != Ls.device or weights.device.type != "cuda":
        raise ValueError("batched mixed LDLQ inputs must share one CUDA device")
    device = weights.device
    if source_indices is None:
        if source_count != batch:
            raise ValueError("batched mixed LDLQ needs one source per member without source_indices")
        sources = list(range(batch))
    else:
        if source_indices.shape != (batch,) or source_indices.dtype != torch.long or source_indices.device != device:
            raise ValueError("mixed LDLQ source_indices must be device-local int64 [B]")
        sources = source_indices.tolist()
        if any(s < 0 or s >= source_count for s in sources):
            raise ValueError("mixed LDLQ source_indices are out of range")
    gathered = source_indices is not None and sources != list(range(source_count))

    multipliers = tuple(enc._ldlq_feedback_multiplier(args) for args in quant_args_list)
    tf32 = bool(quant_args_list[0].get("ldlq_tf32", False))
    if any(bool(args.get("ldlq_tf32", False)) != tf32 for args in quant_args_list):
        raise ValueError("batched mixed LDLQ members must share TF32 policy")
    normalized = [enc.mixed_rate_spec(size_k, size_n, args) for args in quant_args_list]
    rate_axis = normalized[0][0]
    if any(axis != rate_axis for axis, _ in normalized):
        raise ValueError("batched mixed LDLQ members must share one rate axis")
    for args, (_, bits) in zip(quant_args_list, normalized):
        if args.get("mixed_tile_codebook_ids") is not None or args.get("sqg_e4m3_lut_banks_by_bits") is not None:
            raise NotImplementedError("per-tile codebook banks are a research hook outside the B200 hot path")
        if 1 in bits:
            raise NotImplementedError("K1 tiles are outside the B200 tile encoder (K2, K3, K4)")
    tiles_k, tiles_n = size_k // 16, size_n // 16
    buffer_rows = max(quant_args_list[0].get("buf_size_k", 128), 16)
    if any(max(args.get("buf_size_k", 128), 16) != buffer_rows for args in quant_args_list):
        raise ValueError("batched mixed LDLQ members must share one buffer size")
    if buffer_rows % 16 or size_k % buffer_rows:
        raise ValueError("batched mixed LDLQ buffer must tile the EXL K dimension")
    if process_end is None:
        process_end = size_k
    if (
        isinstance(process_begin, bool) or isinstance(process_end, bool)
        or not isinstance(process_begin, int) or not isinstance(process_end, int)
        or not 0 <= process_begin < process_end <= size_k
        or process_begin % buffer_rows or process_end % buffer_rows
    ):
        raise ValueError("mixed LDLQ process interval must be buffer-aligned")
    state = (initial_weights_q, initial_encoded_q, initial_product_cache)
    if any(v is not None for v in state) and not all(v is not None for v in state):
        raise ValueError("mixed LDLQ continuation requires all three state tensors")
    if initial_weights_q is None and process_end != size_k:
        raise ValueError("a lower mixed LDLQ interval requires continuation state")

    weights = weights.contiguous()
    if initial_weights_q is None:
        product_cache = weights.new_zeros((batch, size_k, size_n))
        weights_q = weights.new_zeros((batch, size_k, size_n))
        encoded_q = torch.zeros((batch, tiles_k, tiles_n, 256), dtype=torch.int16, device=device)
    else:
        weights_q, encoded_q, product_cache = initial_weights_q, initial_encoded_q, initial_product_cache
        want, want_enc = (batch, size_k, size_n), (batch, tiles_k, tiles_n, 256)
        if (
            weights_q.shape != want or weights_q.dtype != weights.dtype or weights_q.device != device
            or product_cache.shape != want or product_cache.dtype != weights.dtype or product_cache.device != device
            or encoded_q.shape != want_enc or encoded_q.dtype != torch.int16 or encoded_q.device != device
            or not (weights_q.is_contiguous() and product_cache.is_contiguous() and encoded_q.is_contiguous())
        ):
            raise ValueError("mixed LDLQ continuation state has invalid shape or type")
    # error rows are written by the step that encodes them before any product reads them
    err = torch.empty((batch, size_k, size_n), dtype=torch.float, device=device)
    launches = _Launches(rate_axis, [bits for _, bits in normalized], multipliers, tiles_n, sources, device)
    args0 = quant_args_list[0]

    def pick(block: torch.Tensor) -> torch.Tensor:
        return block.index_select(0, source_indices) if gathered else block

    def gemm(target, a, b):
        allow = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = tf32
        try:
            target.baddbmm_(a, b)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = allow

    # Feedback products on the tensor cores (see encoder._ldlq_steps): the transposed factors are
    # split once per source, the transposed error rows of the current span after every step.
    tensor_cores = bool(args0.get("ldlq_tensor_cores", enc.LDLQ_TENSOR_CORES))
    if tensor_cores:
        from . import linalg

        factor_t = linalg.split_tf32(Ls, transpose=True)
        err_t = linalg.Planes(torch.zeros((batch, size_n, buffer_rows), dtype=torch.float, device=device),
                              torch.zeros((batch, size_n, buffer_rows), dtype=torch.float, device=device))

        def factor_view(rows, cols):
            return linalg.Planes(pick(factor_t.hi[:, rows, cols]), pick(factor_t.lo[:, rows, cols]))

    step = 0
    for end in range(process_end, process_begin, -buffer_rows):
        begin = end - buffer_rows
        for block_end in range(buffer_rows, 0, -16):
            row_begin, row_end = begin + block_end - 16, begin + block_end
            if row_end < end:
                if tensor_cores:
                    linalg.gemm_nt(linalg.Planes(err_t.hi[:, :, block_end:], err_t.lo[:, :, block_end:]),
                                   factor_view(slice(row_begin, row_end), slice(row_end, end)),
                                   product_cache[:, row_begin:row_end], beta=1.0, transposed_out=True)
                else:
                    gemm(product_cache[:, row_begin:row_end],
                         pick(Ls[:, row_end:end, row_begin:row_end]).transpose(1, 2), err[:, row_end:end])
            for launch in launches.at(row_begin // 16):
                _quantize_members(weights, product_cache, weights_q, err, encoded_q, row_begin, launch, args0)
            if tensor_cores:
                linalg.split_tf32(err[:, row_begin:row_end], transpose=True,
                                  out=linalg.Planes(err_t.hi[:, :, block_end - 16:block_end],
                                                    err_t.lo[:, :, block_end - 16:block_end]))
            if pb:
                step += 1
                pb.update(step)
        if begin:
            # rows at or above `begin` are committed; only the rows still to be visited need the
            # span's error folded into their product cache
            if tensor_cores:
                linalg.gemm_nt(factor_view(slice(0, begin), slice(begin, end)), err_t, product_cache[:, :begin], beta=1.0)
            else:
                gemm(product_cache[:, :begin], pick(Ls[:, begin:end, :begin]).transpose(1, 2), err[:, begin:end])
    if tensor_cores:
        linalg.check_status(device)
    if synchronize:
        torch.cuda.synchronize(device)
    if return_product_cache:
        return weights_q, encoded_q, product_cache
    return weights_q, encoded_q


def _check_groups(weights, Ls, quant_args_groups, what: str):
    if weights.ndim != 3 or Ls.ndim != 3:
        raise ValueError(f"{what} expects rank-three weights and Ls")
    source_count, size_k, size_n = weights.shape
    if source_count <= 0 or Ls.shape != (source_count, size_k, size_k):
        raise ValueError(f"{what} weight/L shapes do not agree")
    if len(quant_args_groups) != source_count or any(not group for group in quant_args_groups):
        raise ValueError(f"{what} needs candidates for every source")
    return source_count, size_k, size_n


def _tile_columns(tiles, device) -> torch.Tensor:
    index = torch.tensor(tiles, dtype=torch.int64, device=device)
    return (index[:, None] * 16 + torch.arange(16, device=device)).flatten()


def ldlq_mixed_n_candidates_reuse(weights: torch.Tensor, Ls: torch.Tensor, quant_args_groups: list[list[dict]]):
    """Output-axis candidates from shared encodes (exl3_encoder_backend.py:1481-1642).

    Error feedback couples the rows of the ``[K, N]`` matrix only, so the columns of a candidate
    are encoded independently of one another: the all-K3 first candidate of every source is
    encoded once, the union of K2 columns and the union of K4 columns of its other candidates once
    each, and every candidate is those pieces put side by side.  Returns ``(weight_q, encoded)``
    stacked in source-major candidate order.
    """

    enc = _encoder()
    source_count, size_k, size_n = _check_groups(weights, Ls, quant_args_groups, "output-axis reuse")
    device = weights.device
    maps: list[list[tuple[int, ...]]] = []
    for group in quant_args_groups:
        specs = [enc.mixed_rate_spec(size_k, size_n, args) for args in group]
        if any(axis != "n" for axis, _ in specs):
            raise ValueError("output-axis reuse supports only mixed_rate_axis='n'")
        if specs[0][1] != (3,) * (size_n // 16):
            raise ValueError("output-axis reuse requires an all-K3 first candidate")
        maps.append([bits for _, bits in specs])

    base_q, base_states = ldlq_mixed_batched(weights, Ls, [group[0] for group in quant_args_groups])

    # (source, width) -> tiles that any candidate of that source stores at that width
    unions: list[tuple[int, int, tuple[int, ...]]] = []
    for source, candidate_maps in enumerate(maps):
        width_of: dict[int, int] = {}
        for bits in candidate_maps[1:]:
            for tile, width in enumerate(bits):
                if width != 3 and width_of.setdefault(tile, width) != width:
                    raise ValueError("one output tile uses multiple non-K3 widths across candidates")
        for width in (2, 4):
            tiles = tuple(t for t, w in width_of.items() if w == width)
            if tiles:
                unions.append((source, width, tiles))

    # unions of equal size travel together, K2 and K4 members in the same traversal
    pieces: dict[tuple[int, int], tuple[dict[int, int], torch.Tensor, torch.Tensor]] = {}
    for count in sorted({len(tiles) for _, _, tiles in unions}):
        members = [u for u in unions if len(u[2]) == count]
        member_weights = torch.stack(
            [weights[source].index_select(1, _tile_columns(tiles, device)) for source, _, tiles in members]
        )
        member_args = []
        for source, width, _ in members:
            args = dict(quant_args_groups[source][0])
            args["mixed_tile_bits"] = (width,) * count
            member_args.append(args)
        piece_q, piece_states = _encode_union(member_weights, Ls, [s for s, _, _ in members], member_args)
        for slot, (source, width, tiles) in enumerate(members):
            pieces[(source, width)] = ({tile: i for i, tile in enumerate(tiles)}, piece_q[slot], piece_states[slot])

    out_q, out_states = [], []
    for source, candidate_maps in enumerate(maps):
        for candidate, bits in enumerate(candidate_maps):
            if candidate == 0:
                out_q.append(base_q[source])
                out_states.append(base_states[source])
                continue
            weight_q = base_q[source].clone()
            states = base_states[source].clone()
            for width in (2, 4):
                wanted = tuple(t for t, w in enumerate(bits) if w == width)
                if not wanted:
                    continue
                where, piece_q, piece_states = pieces[(source, width)]
                local = tuple(where[t] for t in wanted)
                weight_q.index_copy_(1, _tile_columns(wanted, device),
                                     piece_q.index_select(1, _tile_columns(local, device)))
                states.index_copy_(1, torch.tensor(wanted, dtype=torch.int64, device=device),
                                   piece_states.index_select(1, torch.tensor(local, dtype=torch.int64, device=device)))
            out_q.append(weight_q)
            out_states.append(states)
    return torch.stack(out_q), torch.stack(out_states)


def _encode_union(member_weights: torch.Tensor, Ls: torch.Tensor, member_sources: list[int], member_args: list[dict]):
    """Column subsets of several sources in one traversal, each member with its source's factor."""

    if member_sources == list(range(Ls.shape[0])):
        return ldlq_mixed_batched(member_weights, Ls, member_args)
    index = torch.tensor(member_sources, dtype=torch.long, device=Ls.device)
    return ldlq_mixed_batched(member_weights, Ls.index_select(0, index), member_args)


def ldlq_mixed_k_candidates_prefix_reuse(weights: torch.Tensor, Ls: torch.Tensor, quant_args_groups: list[list[dict]]):
    """Input-axis candidates with a shared backwards prefix (exl3_encoder_backend.py:1645-1830).

    The traversal runs from the last row upwards, so rate maps that agree on their trailing rows
    share all work down to the first buffer boundary where they part.  That stretch is encoded
    once per source with its product cache kept; from there the live states form a trie: at
    every buffer of rows a state is duplicated once per distinct rate its candidates ask for,
    and all live states advance together in one batched call that reads the immutable sources
    through ``source_indices``.  Returns ``(weight_q, encoded)`` in source-major candidate order.
    """

    enc = _encoder()
    source_count, size_k, size_n = _check_groups(weights, Ls, quant_args_groups, "input-axis prefix reuse")
    if not any(len(group) > 1 for group in quant_args_groups):
        raise ValueError("input-axis prefix reuse needs at least one multi-candidate source")
    device = weights.device
    maps: list[list[tuple[int, ...]]] = []
    first_shared_tile = 0
    for group in quant_args_groups:
        specs = [enc.mixed_rate_spec(size_k, size_n, args) for args in group]
        if any(axis != "k" for axis, _ in specs):
            raise ValueError("input-axis prefix reuse supports only mixed_rate_axis='k'")
        group_maps = [bits for _, bits in specs]
        tile = len(group_maps[0])
        while tile > 0 and len({bits[tile - 1] for bits in group_maps}) == 1:
            tile -= 1
        maps.append(group_maps)
        first_shared_tile = max(first_shared_tile, tile)
    buffer_rows = max(quant_args_groups[0][0].get("buf_size_k", 128), 16)
    if any(max(args.get("buf_size_k", 128), 16) != buffer_rows for group in quant_args_groups for args in group):
        raise ValueError("input-axis prefix reuse requires one LDLQ buffer size")
    # rows [split, size_k) are common to every candidate of every source, on a buffer boundary
    split = -(-(first_shared_tile * 16) // buffer_rows) * buffer_rows
    flat = [(source, candidate) for source, group in enumerate(quant_args_groups) for candidate in range(len(group))]
    flat_sources = torch.tensor([source for source, _ in flat], dtype=torch.long, device=device)

    if split >= size_k:  # nothing in common: plain batch over all candidates
        return ldlq_mixed_batched(weights, Ls, [quant_args_groups[s][c] for s, c in flat], source_indices=flat_sources)

    state_q, state_enc, state_cache = ldlq_mixed_batched(
        weights, Ls, [group[0] for group in quant_args_groups],
        process_begin=split, process_end=size_k, return_product_cache=True, synchronize=False,
    )
    if split == 0:  # the maps agree everywhere
        return state_q.index_select(0, flat_sources), state_enc.index_select(0, flat_sources)

    # a live state = (source, the candidates still following it)
    live = [(source, tuple(range(len(group)))) for source, group in enumerate(quant_args_groups)]
    for end in range(split, 0, -buffer_rows):
        begin = end - buffer_rows
        children, parents, child_args = [], [], []
        for parent, (source, followers) in enumerate(live):
            by_rates: dict[tuple[int, ...], list[int]] = {}
            for candidate in followers:
                by_rates.setdefault(maps[source][candidate][begin // 16:end // 16], []).append(candidate)
            for members in by_rates.values():
                children.append((source, tuple(members)))
                parents.append(parent)
                child_args.append(quant_args_groups[source][members[0]])
        if parents != list(range(len(live))):
            fan_out = torch.tensor(parents, dtype=torch.long, device=device)
            state_q = state_q.index_select(0, fan_out)
            state_enc = state_enc.index_select(0, fan_out)
            state_cache = state_cache.index_select(0, fan_out)
        live = children
        state_q, state_enc, state_cache = ldlq_mixed_batched(
            weights, Ls, child_args, synchronize=False, process_begin=begin, process_end=end,
            initial_weights_q=state_q, initial_encoded_q=state_enc, initial_product_cache=state_cache,
            return_product_cache=True,
            source_indices=torch.tensor([source for source, _ in live], dtype=torch.long, device=device),
        )
    torch.cuda.synchronize(device)
    holder = {(source, candidate): slot for slot, (source, followers) in enumerate(live) for candidate in followers}
    if set(holder) != set(flat):
        raise AssertionError("input-axis prefix trie lost a rate candidate")
    order = torch.tensor([holder[member] for member in flat], dtype=torch.long, device=device)
    return state_q.index_select(0, order), state_enc.index_select(0, order)
