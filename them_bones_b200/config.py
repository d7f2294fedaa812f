"""Configuration: model dataclass, environment switches and recipe files.

Three tiers, as in the reference (round2/source/train.py:80-116 module constants, :365-377 ``_env``,
:3219-3300 ``GPTConfig``/``model_config_dict``, round2/source/final_run.env the sourced recipe):

* ``Hyper``      -- optimizer / schedule / batch constants; every field can be overridden by a ``BONES_*``
                    environment variable of the same upper-cased name.
* ``switches()`` -- feature switches read from the environment once (``BONES_*``); cross-switch validity is
                    checked here and raises before any model is built (reference: launch-time refusals,
                    round2/source/train.py:21449-21508).
* ``GPTConfig``  -- everything the forward pass depends on.  Only non-default fields are serialised into a
                    checkpoint's ``model_config`` so that ``load_for_eval`` rebuilds the model with no environment.

A recipe is a plain ``KEY=VALUE`` file (``recipes/*.env``); ``load_recipe`` applies it to ``os.environ`` without
overriding variables the caller already set, which reproduces ``set -a; . final_run.env`` semantics.
"""
from __future__ import annotations

import os
from dataclasses import MISSING, asdict, dataclass, field, fields

PREFIX = "BONES_"


def _env(name: str, default, kind):
    """Typed environment read.  Booleans accept 0/1/true/false and raise on anything else."""
    raw = os.environ.get(name)
    if raw is None:
        return default
    raw = raw.strip()
    if kind is bool:
        if raw.lower() in ("1", "true"):
            return True
        if raw.lower() in ("0", "false"):
            return False
        raise ValueError(f"{name}={raw!r}: expected 0 or 1")
    if kind is tuple:
        return tuple(int(v) for v in raw.replace(",", " ").split()) if raw else ()
    return kind(raw)


def load_recipe(path: str, override: bool = False) -> dict:
    """Apply a ``KEY=VALUE`` recipe file to ``os.environ``.  Lines starting with ``#`` and blank lines are skipped;
    ``export`` prefixes and surrounding quotes are tolerated.  Returns the pairs that were read."""
    out = {}
    with open(path) as fh:
        for line in fh:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            if line.startswith("export "):
                line = line[len("export "):]
            if "=" not in line:
                raise ValueError(f"{path}: not KEY=VALUE: {line!r}")
            k, v = line.split("=", 1)
            v = v.split(" #", 1)[0].strip().strip('"').strip("'")
            out[k.strip()] = v
    for k, v in out.items():
        if override or k not in os.environ:
            os.environ[k] = v
    return out


@dataclass
class GPTConfig:
    sequence_len: int
    vocab_size: int
    n_layer: int
    n_head: int
    n_embd: int
    head_dim: int = 0              # 0 -> n_embd // n_head
    mlp_ratio: int = 4
    rope_base: float = 100000.0
    qk_scale: float = 0.0          # 0 -> 1/sqrt(head_dim)
    softcap: float = 15.0
    bos_id: int = 0
    doc_mask: bool = False         # causal attention restarts at every BOS token
    unet: bool = False             # U-net skips between the first and last n_layer//2 blocks
    value_embeds: int = 0          # number of value-embedding tables on alternating last layers
    attn_window: int = 0           # sliding window in tokens (multiple of 128) on the layers not in attn_long
    attn_long: tuple = ()          # layers that keep full causal attention when attn_window > 0
    attn_layers: tuple = ()        # blocks that have attention (empty: all); the others are MLP-only
    mixer: str = "off"             # "shift1": attention-free blocks add mix_lambda * (x shifted by one token)
    mtp_offsets: tuple = ()        # extra next-token targets, e.g. (2, 3): predict t+2 and t+3 from position t
    label_smoothing: float = 0.0   # training loss only; evaluation is the plain cross-entropy
    mlp_precision: str = "bf16"    # "bf16" | "mxfp8": block-scaled MLP / expert GEMMs
    attn_proj_precision: str = "bf16"   # "bf16" | "mxfp8": block-scaled qkv / out projections (attention core stays bf16)
    moe_layers: tuple = ()
    moe_experts: int = 0
    moe_topk: int = 0
    moe_capacity: int = 0          # assignments one expert serves within one sequence
    moe_hidden: int = 0
    moe_shared: int = 0            # hidden width of the always-on shared MLP half (0: none)
    moe_aux: float = 0.01
    moe_zloss: float = 0.0
    table_orders: tuple = ()       # hashed n-gram input tables, e.g. (2, 3)
    table_rows: int = 0            # rows per table (power of two)
    table_seed: int = 0
    table_bits: int = 0            # 1 or 4: every read takes a packed view of the row (0: the row itself)
    # output-side hashed table (0 rows: off): keyed by the os1_order ids ending at a position; its sign-hashed row is read
    # out through a fixed codebook and added to the logits before the soft-cap (reference: switch 59,
    # round2/source/train.py:2310-2351; the defaults below are the reference's)
    os1_rows: int = 0
    os1_dim: int = 128
    os1_order: int = 16
    os1_lr: float = 0.125           # the read-out scale is os1_a0 * os1_lr, so the step size belongs to the model
    os1_a0: float = 7.98
    os1_thr: float = 0.7
    os1_beta: float = 3.0
    os1_glin: float = 0.01
    os1_gate_w: int = 32
    os1_gate_h0: float = 0.3
    os1_gate_slope: float = 30.0
    os1_seed: int = 0
    os1_code_seed: int = 5901
    os1_bits: int = 0              # 1: every read takes the row's 1-bit view sign(m) * mean|m|

    def __post_init__(self):
        for name in ("attn_long", "moe_layers", "table_orders", "attn_layers", "mtp_offsets"):
            setattr(self, name, tuple(int(v) for v in getattr(self, name)))
        if self.head_dim == 0:
            self.head_dim = self.n_embd // self.n_head
        if self.attn_window and self.attn_window % 128:
            raise ValueError("attn_window must be a multiple of the 128-token attention tile")
        if self.mixer not in ("off", "shift1"):
            raise ValueError(f"mixer={self.mixer!r}: expected 'off' or 'shift1'")
        if any(o < 2 for o in self.mtp_offsets):
            raise ValueError("mtp_offsets are distances beyond the next token: each must be >= 2")
        if self.mlp_precision not in ("bf16", "mxfp8"):
            raise ValueError(f"mlp_precision={self.mlp_precision!r}")
        if self.attn_proj_precision not in ("bf16", "mxfp8"):
            raise ValueError(f"attn_proj_precision={self.attn_proj_precision!r}")
        if self.moe_layers:
            if not (self.moe_experts and self.moe_topk in (1, 2) and self.moe_capacity and self.moe_hidden):
                raise ValueError("MoE layers need moe_experts, moe_topk in {1,2}, moe_capacity and moe_hidden")
        if self.table_orders and (self.table_rows & (self.table_rows - 1) or self.table_rows <= 0):
            raise ValueError("table_rows must be a positive power of two")
        if self.table_bits not in (0, 1, 4) or self.os1_bits not in (0, 1):
            raise ValueError("table_bits is 0, 1 or 4 and os1_bits 0 or 1")
        if (self.table_bits and self.n_embd % 8) or (self.os1_bits and self.os1_dim % 8):
            raise ValueError("packed views need a row width that is a multiple of 8")
        if self.os1_rows and (self.os1_rows & (self.os1_rows - 1) or self.os1_dim % 32 or self.os1_dim > 256):
            raise ValueError("os1_rows must be a power of two and os1_dim a multiple of 32 up to 256")

    @property
    def padded_vocab(self) -> int:
        return -(-self.vocab_size // 64) * 64

    @property
    def attn_dim(self) -> int:
        return self.n_head * self.head_dim


def model_config_dict(config: GPTConfig) -> dict:
    """``asdict`` without fields at their defaults (reference: round2/source/train.py:3289-3296)."""
    out = asdict(config)
    for f in fields(GPTConfig):
        if f.default is not MISSING and out[f.name] == f.default:
            del out[f.name]
    if out.get("head_dim") == config.n_embd // config.n_head:
        out.pop("head_dim", None)
    return {k: (list(v) if isinstance(v, tuple) else v) for k, v in out.items()}


def moe_capacity_for(cf: float, seq_len: int, topk: int, n_exp: int) -> int:
    """C = round(cf * T * k / E), at least 1 (reference: round2/source/train.py:10482-10484)."""
    return max(1, int(round(cf * seq_len * topk / n_exp)))


def parse_layers(spec: str, depth: int) -> tuple:
    """``"2:"`` / ``"9,11,13"`` / ``"odd"`` / ``"all"`` -> tuple of layer ids (reference: ``parse_moe_layers``,
    round2/source/train.py:10463)."""
    spec = spec.strip()
    if not spec or spec == "none":
        return ()
    if spec == "all":
        return tuple(range(depth))
    if spec == "odd":
        return tuple(i for i in range(depth) if i % 2 == 1)
    if spec.endswith(":"):
        return tuple(range(int(spec[:-1]), depth))
    out = tuple(sorted({int(v) for v in spec.replace(",", " ").split()}))
    if out and (out[0] < 0 or out[-1] >= depth):
        raise ValueError(f"layer list {spec!r} outside 0..{depth - 1}")
    return out


@dataclass
class Hyper:
    """Optimizer, schedule and batch constants (reference defaults: round2/source/train.py:80-116 and
    round2/submission/train.py:157-226; Appendix values of the final recipe)."""
    total_batch: int = 524288          # tokens per optimizer step over all ranks
    device_batch: int = 8              # sequences per micro-step per rank
    embedding_lr: float = 0.30
    unembedding_lr: float = 0.006
    matrix_lr: float = 0.025
    scalar_lr: float = 0.20
    resid_lr_div: float = 28.0         # resid_lambda trains at scalar_lr / resid_lr_div
    table_lr: float = 0.02
    os1_cap: float = 4.0               # output table: a row's RMS stays below os1_cap * os1_lr
    os1_eps_rel: float = 1e-6          # ... and eps of its normalised step, relative to a typical one-position gradient
    weight_decay: float = 0.05
    warmup_steps: int = 40
    warmdown_frac: float = 0.85
    final_lr_frac: float = 0.01
    rows_warmdown_frac: float = 0.65
    rows_final_lr_frac: float = 0.05
    muon_momentum: float = 0.95
    muon_beta2: float = 0.90
    ns_steps: int = 5
    moe_lr: float = 0.025
    moe_cf: float = 1.25
    seed: int = 42
    bad_loss: float = 100.0
    rescue_from: float = 0.85
    rescue_every: int = 200
    log_every: int = 10
    sync_every: int = 100              # forced synchronous step boundary
    startup_steps_excluded: int = 5

    @classmethod
    def from_env(cls) -> "Hyper":
        h = cls()
        for f in fields(cls):
            setattr(h, f.name, _env(PREFIX + f.name.upper(), getattr(h, f.name), type(getattr(h, f.name))))
        return h


_SWITCHES = None


def switches(refresh: bool = False) -> dict:
    """Feature switches as run.  The returned dict is recorded in a checkpoint's ``meta`` (reference:
    ``recipe_switches``, round2/source/train.py:1043)."""
    global _SWITCHES
    if _SWITCHES is not None and not refresh:
        return _SWITCHES
    e = lambda n, d, k: _env(PREFIX + n, d, k)  # noqa: E731
    s = dict(
        # model
        UNET=e("UNET", False, bool), VE=e("VE", 0, int), QK_SCALE=e("QK_SCALE", 0.0, float),
        ROPE_BASE=e("ROPE_BASE", 100000.0, float), DOC_MASK=e("DOC_MASK", False, bool),
        ATTN_WINDOW=e("ATTN_WINDOW", 0, int), ATTN_LONG=e("ATTN_LONG", "", str),
        ATTN_LAYERS=e("ATTN_LAYERS", "", str), MIXER=e("MIXER", "off", str), MLP_RATIO=e("MLP_RATIO", 4, int),
        LABEL_SMOOTH=e("LABEL_SMOOTH", 0.0, float), MTP=e("MTP", "", str), MTP_WEIGHT=e("MTP_WEIGHT", 0.5, float), MTP_ANNEAL=e("MTP_ANNEAL", 0.5, float),
        MLP=e("MLP", "bf16", str),
        ATTN_PROJ=e("ATTN_PROJ", "bf16", str),       # bf16 | mxfp8: the attention projections' GEMMs and weight gradients
        MOE=e("MOE", False, bool), MOE_LAYERS=e("MOE_LAYERS", "", str), MOE_EXPERTS=e("MOE_EXPERTS", 16, int),
        MOE_TOPK=e("MOE_TOPK", 2, int), MOE_HIDDEN=e("MOE_HIDDEN", 0, int), MOE_SHARED=e("MOE_SHARED", 0, int),
        MOE_AUX=e("MOE_AUX", 0.01, float), MOE_ZLOSS=e("MOE_ZLOSS", 0.0, float),
        TABLES=e("TABLES", "", str), TABLE_ROWS=e("TABLE_ROWS", 0, int), TABLE_SEED=e("TABLE_SEED", 0, int), TABLE_BITS=e("TABLE_BITS", 0, int), OS1_BITS=e("OS1_BITS", 0, int),
        TABLE_HOST_STATE=e("TABLE_HOST_STATE", "auto", str),   # auto | 0 | 1: Adam moments of the tables in pinned host memory
        TABLE_OPT=e("TABLE_OPT", "auto", str),       # auto | adam | rowrms (one fp32 second moment per row)
        OS1=e("OS1", False, bool), OS1_ROWS=e("OS1_ROWS", 1 << 24, int), OS1_ORDER=e("OS1_ORDER", 16, int),
        OS1_LR=e("OS1_LR", 0.125, float), OS1_SEED=e("OS1_SEED", 0, int),
        # answer phase: from progress 1 - ANSWER_PHASE on, the loader marks the last ANSWER_TAIL of every document and the
        # loss weights those targets by ANSWER_WEIGHT (reference: switch 29, QaPhase round2/source/train.py:19691)
        ANSWER_PHASE=e("ANSWER_PHASE", 0.0, float), ANSWER_TAIL=e("ANSWER_TAIL", 0.25, float),
        ANSWER_WEIGHT=e("ANSWER_WEIGHT", 2.0, float),
        EVAL_SPLIT=e("EVAL_SPLIT", False, bool),     # after the final evaluation: held-out loss by position class
        DATA_RULE=e("DATA_RULE", "", str),           # e.g. "len:64-4096,band:0.05-0.95,dedup:32,from:0.1"
        # riders of the packer (data/streams.py), e.g. "pool:0.1@0.3x2,strata:0.05@0.3,blocks:0.02+late,edge,dedup:/dev/shm/d"
        DATA_STREAMS=e("DATA_STREAMS", "", str),
        # kernels / system
        SELFCHECK=e("SELFCHECK", False, bool),       # compare every native op with the PyTorch path before training
        KERNELS=e("KERNELS", "auto", str),           # auto: CUDA kernels on a GPU, torch oracle on CPU | ref
        FUSED_COMM=e("FUSED_COMM", True, bool),      # in-kernel NVLink collectives (False: NCCL baseline path)
        # fused reductions / publishes through NVSwitch multicast (multimem.ld_reduce / multimem.st) where the slab has a
        # mapping.  Off by default: for a reduce-scatter every GPU still uploads its copy of the others' chunks, so the
        # links carry the same bytes as with peer loads (measured on 4 GPUs: 1.97 against 1.82 ms for the Muon slabs)
        NVLS=e("NVLS", False, bool),
        WGRAD_PUSH=e("WGRAD_PUSH", False, bool),     # weight-gradient GEMMs reduce-scatter their tiles into the owner's slab
        LOSS_ROWS=e("LOSS_ROWS", 4096, int),         # rows per block of the chunked loss head (one [rows, V] logits buffer)
        GRAD_CLIP=e("GRAD_CLIP", 0.0, float),        # > 0: global-norm clip of the reduced gradients (library-collective path)
        MASTER=e("MASTER", "fp32", str),             # fp32 | bf16: Muon master copies (bf16 = stochastic rounding)
        OPT=e("OPT", "lean", str),                   # lean | dist | single
        OPT_OVERLAP_CHECK=e("OPT_OVERLAP_CHECK", False, bool),
        FINITE_GATE=e("FINITE_GATE", True, bool),
        BOUNDARY_ASYNC=e("BOUNDARY_ASYNC", True, bool),
        PREFETCH=e("PREFETCH", True, bool),
        SHED=e("SHED", False, bool),
        SEQ_RAMP=e("SEQ_RAMP", 0.0, float),           # clock fraction trained on half-length windows
        EMA=e("EMA", 0.0, float),
        MEM_PRINT=e("MEM_PRINT", False, bool), MEM_PHASE=e("MEM_PHASE", -1, int),
        MICRO_BARRIER=e("MICRO_BARRIER", False, bool),
        SAVE_OPT_STATE=e("SAVE_OPT_STATE", False, bool),
        SAVE_EVERY=e("SAVE_EVERY", 0, int),          # > 0: a checkpoint every so many steps, written on a background thread
    )
    if s["MLP"] not in ("bf16", "mxfp8"):
        raise ValueError(f"{PREFIX}MLP={s['MLP']!r}: expected bf16 or mxfp8")
    if s["KERNELS"] not in ("auto", "ref"):
        raise ValueError(f"{PREFIX}KERNELS={s['KERNELS']!r}: expected auto or ref")
    if s["OPT"] not in ("lean", "dist", "single"):
        raise ValueError(f"{PREFIX}OPT={s['OPT']!r}")
    if s["MOE_TOPK"] not in (1, 2):
        raise ValueError(f"{PREFIX}MOE_TOPK must be 1 or 2")
    if s["SHED"] and s["MOE"]:
        # a rank that drops a micro-batch would leave its peers' expert all-to-all one call short
        raise ValueError("straggler shedding is refused with MoE (reference: round2/source/train.py:3035-3038)")
    if s["ATTN_WINDOW"] % 128:
        raise ValueError(f"{PREFIX}ATTN_WINDOW must be a multiple of 128")
    _SWITCHES = s
    return s


def build_config(depth: int, n_embd: int, n_head: int, seq_len: int, vocab: int, *, head_dim: int = 0,
                 bos_id: int = 0, hyper: Hyper | None = None) -> GPTConfig:
    """Geometry from the CLI + switches from the environment -> GPTConfig (reference: ``build_config``,
    round2/source/train.py:11718-11757)."""
    s = switches()
    h = hyper or Hyper.from_env()
    kw = dict(sequence_len=seq_len, vocab_size=vocab, n_layer=depth, n_head=n_head, n_embd=n_embd, head_dim=head_dim,
              rope_base=s["ROPE_BASE"], qk_scale=s["QK_SCALE"], bos_id=bos_id, doc_mask=s["DOC_MASK"], unet=s["UNET"],
              value_embeds=s["VE"], attn_window=s["ATTN_WINDOW"], mlp_precision=s["MLP"], attn_proj_precision=s["ATTN_PROJ"],
              mlp_ratio=s["MLP_RATIO"],
              mixer=s["MIXER"], label_smoothing=s["LABEL_SMOOTH"])
    if s["ATTN_LAYERS"]:
        kw["attn_layers"] = parse_layers(s["ATTN_LAYERS"], depth)
    if s["MTP"]:
        kw["mtp_offsets"] = tuple(int(v) for v in s["MTP"].split(",") if v.strip())
    if s["ATTN_WINDOW"]:
        kw["attn_long"] = (parse_layers(s["ATTN_LONG"], depth) if s["ATTN_LONG"]
                           else tuple(i for i in range(depth) if i % 4 == 3 or i == depth - 1))
    if s["MOE"]:
        layers = parse_layers(s["MOE_LAYERS"] or "2:", depth)
        kw.update(moe_layers=layers, moe_experts=s["MOE_EXPERTS"], moe_topk=s["MOE_TOPK"],
                  moe_capacity=moe_capacity_for(h.moe_cf, seq_len, s["MOE_TOPK"], s["MOE_EXPERTS"]),
                  moe_hidden=s["MOE_HIDDEN"] or 2 * n_embd, moe_shared=s["MOE_SHARED"], moe_aux=s["MOE_AUX"],
                  moe_zloss=s["MOE_ZLOSS"])
    if s["TABLES"]:
        kw.update(table_orders=_env(PREFIX + "TABLES", (), tuple), table_rows=s["TABLE_ROWS"] or (1 << 20),
                  table_seed=s["TABLE_SEED"], table_bits=s["TABLE_BITS"])
    if s["OS1"]:
        kw.update(os1_rows=s["OS1_ROWS"], os1_order=s["OS1_ORDER"], os1_lr=s["OS1_LR"], os1_seed=s["OS1_SEED"], os1_bits=s["OS1_BITS"])
    return GPTConfig(**kw)


def micro_batch_for(total_batch: int, world: int, preferred: int, seq_len: int) -> int:
    """Sequences per micro-step per rank: the largest value not above ``preferred`` that divides the rank's share of the
    global batch (with a fixed global batch the share shrinks as ranks are added)."""
    share = max(1, total_batch // (seq_len * world))
    db = max(1, min(preferred, share))
    while share % db:
        db -= 1
    return db


# Named model geometries of the five benchmark configurations.
GEOMETRY = {
    "tiny": dict(depth=4, n_embd=256, n_head=4, seq_len=256, vocab=8192),
    "round1": dict(depth=20, n_embd=1280, n_head=10, seq_len=2048, vocab=65536),
}
