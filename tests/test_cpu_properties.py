"""Property tests (hypothesis) of the host-side rules that the kernels and the distributed plumbing rely on: the MX
block-scale rule and its rounding, the scale-chunk layout that the quantiser writes and the GEMM's TMA reads, the
placement of Muon matrices over ranks, batch arithmetic, document starts, and the packer and its riders on ragged
inputs."""
import numpy as np
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

FAST = settings(max_examples=40, deadline=None)


@FAST
@given(st.integers(1, 6), st.integers(1, 4), st.floats(-30, 30), st.integers(0, 2 ** 31 - 1))
def test_mx_quantisation_never_saturates_and_its_error_is_bounded_per_block(rows, blocks, log_scale, seed):
    """Scales are powers of two chosen so that a block's largest magnitude lands in (224, 448]; the round trip is exact
    for zeros and within half an E4M3 step of the block's largest magnitude elsewhere."""
    from them_bones_b200.ref import functional as RF
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, blocks * 32, generator=g) * 2.0 ** log_scale).bfloat16().float()
    x[0, :32] = 0
    q, e = RF.mx_quantize(x, -1)
    scale = torch.exp2(e.float() - 127.0)
    amax = x.view(rows, blocks, 32).abs().amax(-1)
    scaled = amax / scale
    live = amax > 0
    assert bool((scaled[live] <= 448.0).all()) and bool((scaled[live] > 224.0 - 1e-3).all())
    assert bool((e[~live] == 0).all())
    back = RF.mx_dequantize(q, e, -1)
    err = (back - x).view(rows, blocks, 32).abs().amax(-1)
    assert bool((err <= amax * 2.0 ** -4 + 1e-30).all())              # three mantissa bits: half a step of 2^-3
    assert bool((back[0, :32] == 0).all())


def _sf_offset(r, k, kblocks, group):
    """The scale-chunk layout (csrc/gemm_mxfp8_2cta.cu::q_sf_offset): tiles of ``group`` rows, K blocks of 128, chunks of
    128 rows x 4 scales as 32 x 16 bytes."""
    g, t = divmod(r, group)
    chunks = (group + 127) // 128
    return ((g * kblocks + (k >> 7)) * chunks + (t >> 7)) * 512 + (t & 31) * 16 + ((t & 127) >> 5) * 4 + ((k & 127) >> 5)


@FAST
@given(st.integers(1, 700), st.integers(1, 6), st.sampled_from([128, 160, 224, 256]))
def test_scale_chunk_layout_is_a_bijection_into_the_buffer(rows, kblocks, group):
    """Every (row, 32-wide block) of an operand owns one byte of the scale buffer, inside ``sf2_bytes`` and shared with
    no other; the 32 rows of a row block of the quantiser differ by 16 bytes, a K block's four scales are adjacent."""
    from them_bones_b200.ops.mxfp8 import sf2_bytes
    k = kblocks * 128
    total = sf2_bytes(rows, k, group)
    offs = np.array([[_sf_offset(r, kk, kblocks, group) for kk in range(0, k, 32)] for r in range(rows)])
    assert offs.min() >= 0 and offs.max() < total
    assert len(np.unique(offs)) == offs.size
    assert (np.diff(offs.reshape(rows, kblocks, 4), axis=2) == 1).all()
    r0 = (rows // 32) * 32
    if r0 >= 32 and group % 32 == 0:
        blk = offs[r0 - 32:r0, 0]
        assert (np.diff(blk) == 16).all()


@FAST
@given(st.lists(st.tuples(st.integers(1, 90), st.sampled_from([(256, 256), (1024, 256), (256, 1024), (1280, 5120)])), min_size=1,
                max_size=5), st.integers(1, 16))
def test_muon_placement_covers_every_matrix_once_and_balances_the_work(groups, world):
    from them_bones_b200.optim.lean import plan_muon_counts
    shapes = [(n, r, c) for n, (r, c) in groups]
    plan = plan_muon_counts(shapes, world)
    load = np.zeros(world)
    for (n, r, c), counts in zip(shapes, plan):
        k = -(-n // world)
        assert len(counts) == world and sum(counts) == n and max(counts) <= k and min(counts) >= n // world
        load += np.asarray(counts) * (r * c * min(r, c))
    heaviest = max(r * c * min(r, c) for _, r, c in shapes)
    assert load.max() - load.min() <= heaviest * len(shapes)          # no rank is more than one matrix per group ahead


@FAST
@given(st.integers(1, 64), st.sampled_from([1, 2, 3, 4, 8]), st.integers(1, 64), st.sampled_from([256, 2048]))
def test_micro_batch_divides_the_ranks_share(seqs_per_rank, world, preferred, seq_len):
    from them_bones_b200.config import micro_batch_for
    total = seqs_per_rank * world * seq_len
    db = micro_batch_for(total, world, preferred, seq_len)
    assert 1 <= db <= preferred and seqs_per_rank % db == 0
    assert all(seqs_per_rank % d for d in range(db + 1, min(preferred, seqs_per_rank) + 1))   # the largest such value


@FAST
@given(st.integers(1, 4), st.integers(2, 96), st.integers(0, 2 ** 31 - 1))
def test_document_starts_point_at_the_latest_bos(b, t, seed):
    from them_bones_b200.ref import functional as RF
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 4, (b, t), generator=g)                     # id 0 is BOS: frequent
    ds = RF.doc_start_positions(idx, 0)
    for i in range(b):
        last = 0
        for j in range(t):
            if int(idx[i, j]) == 0:
                last = j
            assert int(ds[i, j]) == last


@FAST
@given(st.integers(2, 6), st.sampled_from([64, 128]), st.integers(0, 10 ** 6), st.floats(0.0, 0.3))
def test_packed_rows_with_riders_keep_ids_valid_and_mask_what_must_not_train(windows, seq_len, seed, share):
    """Rows of any geometry, with masked blocks and the edge re-lay riding on the packer: inputs are valid ids, every
    target is -1 or a valid id, BOS and masked ids are never targets, and a window's targets are its inputs shifted."""
    from them_bones_b200.data.streams import Streams
    from them_bones_b200.data.synth import PackedRows, ZipfDocs, slice_windows
    from them_bones_b200.data.streams import decode_row
    vocab = 512
    spec = (f"blocks:{share:.3f}," if share > 0.01 else "") + "edge"
    streams = Streams.parse(spec, vocab=vocab, seq_len=seq_len, seed=seed)
    rows = PackedRows(ZipfDocs(vocab, doc_len=(8, 3 * seq_len), seed=seed), windows * seq_len, buffer_docs=64, streams=streams)
    for _ in range(3):
        row = rows.next_row()
        assert len(row) == windows * seq_len + 1
        ids, trainable = decode_row(row)
        x, y = slice_windows(row, seq_len, 0)
        assert x.shape == (windows, seq_len) and int(x.min()) >= 0 and int(x.max()) < vocab
        flat_y, nxt = y.reshape(-1), ids[1:windows * seq_len + 1]
        keep = flat_y >= 0
        assert (flat_y[keep] == nxt[keep]).all() and (flat_y[~keep] == -1).all()
        assert not keep[(nxt == 0) | ~trainable[1:windows * seq_len + 1]].any()


@FAST
@given(st.lists(st.integers(3, 400), min_size=3, max_size=40), st.sampled_from([64, 128, 256]), st.integers(0, 10 ** 6))
def test_edge_relay_permutes_whole_pieces_only(lengths, window, seed):
    from them_bones_b200.data.streams import EdgeRelay
    rng = np.random.default_rng(seed)
    pieces = []
    for n in lengths:
        p = rng.integers(1, 500, size=n).astype(np.int64)
        p[0] = 0
        if rng.random() < 0.3:                                         # a block: some masked ids
            p[1:1 + n // 2] = -(p[1:1 + n // 2] + 1)
        pieces.append(p)
    row = np.concatenate(pieces)
    out = EdgeRelay(window).relay(row)
    split = lambda r: [tuple(x) for x in np.split(r, np.flatnonzero(np.where(r < 0, -r - 1, r) == 0)[1:])]  # noqa: E731
    a, b = split(row), split(out)
    assert sorted(a) == sorted(b) and a[-1] == b[-1] and len(out) == len(row)
