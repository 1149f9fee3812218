"""Typed configuration for the memarch model family, the Instinct optimizer and a training run.

The reference configures itself through ~150 environment variables read at import or constructor time
(full2.py:1270-1429, fastloop.py:52-60, exp_opt.py:182-334).  Here every knob is a dataclass field; `from_env`
maps the reference's variable names onto the fields so a user's existing launch recipes keep working, and
`preset(name)` reproduces the model-name grammar of `lm.build` / `build_full2` (lm.py:752-807, full2.py:2000-2058).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass
class MemoryConfig:
    """Fresh/dim card memory (mem2.py:51-73 constructor arguments)."""
    fresh: int = 64
    dim: int = 192
    dim_max: int = 256
    faces: int = 2
    d_face: int = 64
    d_dim: Optional[int] = None
    write: int = 32
    focus: int = 8
    match: float = 0.8
    w_use: float = 2.0
    w_age: float = 1e-3
    volume: bool = False          # mem3.VolumeMemory
    lean: bool = True             # MEM_LEAN: content projection only for the selected words


@dataclass
class ModelConfig:
    vocab: int = 50304
    d: int = 1024
    heads: int = 16
    light_a: int = 2
    light_b: int = 2
    heavy: int = 14
    final: int = 2
    frac: float = 0.2             # target anchor share (ANCHOR_FRAC)
    cap: float = 0.25             # per-text anchor ceiling (ANCHOR_CAP)
    window: int = 2048
    seg: int = 512
    ckpt: str = ""                # "", "1", "heavy", "light" activation recompute
    use_memory: bool = True       # False: memory reads zeroed (honest-task control, *_nomem)
    no_mem: bool = False          # NO_MEM: memory and reread skipped entirely
    no_reread: bool = False
    memory: MemoryConfig = field(default_factory=MemoryConfig)
    # heavy layers
    moe: str = ""                 # "", "fixed", "budget"
    wave: str = ""                # "", "err", "still"
    n_exp: int = 8
    n_frozen: int = 0             # static frozen tail (Fv2moeE<E>f<pct>)
    bank: bool = False            # BankMoE: waves + real frozen bank
    moe_k: int = 2                # MOE_K
    moe_act: str = "swiglu"       # "swiglu" | "relu2" (MOE_ACT)
    bf16_experts: bool = False    # BF16_EXPERTS
    bank_q: str = ""              # "", "int8", "int4" storage of the frozen bank
    wave_warm: int = 500          # WAVE_WARM
    wave_every: int = 50
    hint_w: float = 1.0
    students: int = 5
    err_thr: float = 0.3
    moe_cap_align: int = 0        # MOE_CAP_ALIGN
    moe_dropless: bool = False    # MOE_GMM: no token is dropped (a place for every anchor in every expert; padding costs no GEMM work)
    moe_group: int = 512
    layer_stats: bool = False     # LAYER_STATS: per-layer MoE statistics (dropped share, experts in use) and the mean fill
    heavy_attn: bool = False
    heavy_attn_detach: bool = False
    n_draft: int = 0
    draft_loss: float = 0.0
    # "instinct on words" (INST_WORD=1): nothing extra for a word guessed well (p >= iw_ok); a gentle push of the right
    # word up to iw_target where the distribution is smeared (leader < iw_spread); the one wrong word the model is sure
    # of (leader != target, p > iw_cw) is pressed down to iw_cw, no further
    inst_word: bool = False
    iw_ok: float = 0.5
    iw_spread: float = 0.35
    iw_target: float = 0.3
    iw_spread_w: float = 0.2
    iw_cw: float = 0.5
    iw_cw_w: float = 0.1
    iw_rewrite: bool = False      # IW_REWRITE: the rewritten answer as target: the right word +delta, its top competitors -delta
    iw_delta: float = 0.05
    iw_random: bool = False       # IW_RANDOM: -delta goes to one random word per row instead (no top-k)
    iw_k: int = 4
    norm_dump_proj: bool = False  # NORM_DUMP_PROJ: the final norm removes the component along the stream's common direction
    safe_norm_ratio: float = 0.0  # SAFE_NORM_RATIO: after the final norm the common vector is capped at ratio x the words' signal
    safe_norm_t0: int = 256
    hn_guard_w: float = 0.0       # HN_GUARD_W: hinge penalty on the trunk: |row mean of hn| > hn_guard_mean or mean |hn| > hn_guard_len
    hn_guard_mean: float = 15.0
    hn_guard_len: float = 42.0
    attn_gain: float = 1.0        # ATTN_GAIN: multiplier of the light blocks' attention scores
    prev_in: bool = False         # PREV_IN: every word also receives the previous word's input vector through a learned gate
    heavy_rotate: bool = False    # HEAVY_ROTATE: every heavy_full_every-th step one heavy layer (in rotation) runs on ALL words
    heavy_full_every: int = 1
    heavy_all: bool = False       # HEAVY_ALL: every heavy layer on all words (last phase / finished model)
    # layer pool (models/fishki.py::FishPool): the heavy MoE layers are replaced by fish_n equal FFN layers; every step
    # is one kind of text and runs through a combination of fish_c layers of that kind's set (FISH_N=<n>)
    fish_n: int = 0
    fish_hf: int = 1024           # width of one layer
    fish_kinds: int = 5
    fish_pool: int = 17           # layers in a kind's set
    fish_c: int = 2               # layers per training step
    fish_eval: bool = False       # finished model: the router picks each row's kind, the row runs the whole set
    fish_eval_c: int = 0          # ... or a fixed subset of this many layers of the set
    fish_center: bool = False     # a layer's input without the stream's common vector
    # "hoop" (models/fishki.py::Uroboros): the heavy layers get the words where the model itself expects to be wrong -
    # a small head predicts the model's own loss per word - instead of the light head's surprise against a threshold
    uroboros: bool = False        # UROBOROS=1
    uroboros_budget: float = 0.25  # share of words sent to the heavy layers (hard top-k)
    uroboros_levels: Tuple[float, ...] = (0.25, 0.18, 0.12, 0.08)   # budgets the loop may step down through
    uroboros_eat: float = 1.0     # a word counts as "eaten" when its predicted loss is below this many nats
    uroboros_w: float = 0.1       # weight of the head's squared error in the loss
    uroboros_thr: float = -1.0    # >= 0: causal choice (evaluation): a word goes heavy when its prediction exceeds this
    uroboros_at: str = "light_b"  # where the head reads: "light_b" (after the memory point) | "light_a" (before)
    # anchor-routed long-range read ("tether", models/rope_memory.py) in the light blocks after the memory point,
    # instead of the segment memory and the re-reading (ROPE_MEM=1; sets no_mem)
    rope_mem: bool = False
    rope_k: int = 4               # anchors a query opens
    rope_links: int = 8           # keys that represent an anchor in the search
    rope_win: int = 64            # local window of the tethered layers
    rope_span_cap: int = 256
    rope_route: str = "hier"      # "hier" | "exact"
    rope_hier_g: int = 64
    rope_hier_nb: int = 16
    rope_hier_bm: int = 64
    rope_excl_win: bool = True
    rope_rgrad: bool = True
    rope_chunk: int = 256
    rope_layers: int = 0          # how many of the first light_b layers are tethered (0: all)
    rope_share_route: bool = False  # later layers reuse the first layer's choice of anchors
    rope_tau0: float = 5.0        # initial surprise threshold of the tether's anchors
    rope_frac: float = 0.0        # share of words that become tether anchors (0: the heavy anchors' share)
    rope_cap: float = 0.0         # ceiling of tether anchors as a share of T (0: the heavy anchors' ceiling)
    rope_anchor_top: bool = False  # over the ceiling keep the most surprising anchors, not the first ones
    rope_qfrac: float = 1.0       # share of words that read the tether at all (the rest: window only)
    rope_qtau0: float = 5.0
    rope_doc_eos: int = -1        # >= 0: anchors of another document than the query's are not opened
    rope_route_bf16: bool = False  # ROPE_ROUTE_BF16: exact search on bf16 operands: tensor-core scores + top-k kernel on a GPU
    rope_pcut: float = 0.0        # ROPE_PCUT: tethered layers rotate only frequencies with a wavelength <= this many words
    rope_key_diag: bool = False   # statistics: how many needle keys the search can see
    remind_use_w: float = 0.0     # REMIND_USE_W: penalty mean(1 - tether share) on the needle questions
    # loss on the answers of recall needles (data.reminders); 0 = the batch's "rem" mask is only scored, not trained on
    remind_w_synth: float = -1.0  # REMIND_W_SYNTH: the weight on synthetic steps (-1: remind_w); lets the text weight move alone
    remind_w: float = 0.0         # REMIND_W: weight of the term (sum of the answers' NLL / (B * remind_q))
    remind_q: int = 16            # questions per needle row (the normaliser)
    remind_cap: int = 0           # answers read per row (0: remind_q); more with several needles per row
    remind_mean: bool = False     # REMIND_MEAN: mean over the batch's answers (episode rows have many)
    remind_only: bool = False     # REMIND_ONLY: stage one, the main loss does not train
    remind_cand: bool = False     # REMIND_CAND: softmax over the 64 value tokens only
    remind_mask_main: bool = False  # REMIND_MASK_MAIN: needle tokens do not train the main loss
    remind_strict: bool = False   # REMIND_STRICT: nothing earned after a row's first wrong answer + penalty on guessing
    remind_strict_w: float = 1.0
    remind_tok0: int = 1000       # REMIND_TOK0: first needle token (keys 512, values 64, marker)
    # light block variants (BLK set)
    blk: Tuple[str, ...] = ()     # subset of {zero, ve, x0, relu2, relu2c, qk, qkv3, smear}
    light_ffn: float = 0.0        # LIGHT_FFN width in units of d
    light_moe: str = ""           # "E:k"
    rope_half: bool = False
    resid_bf16: bool = False
    # phrasebook / locks / heads
    phrase_init: str = ""         # path of the PPMI-SVD artefact
    phrase_c: float = 0.05
    surp_phrase: bool = False
    phrase3: str = ""             # bigram -> next phrase table artefact
    phr_hash: bool = False
    phr_v: int = 50257
    phrase4: str = ""
    skip: str = ""
    skip_g: float = 0.25
    tongue: str = ""
    tongue_a: float = 0.5
    induct: str = ""              # "", "1", "lock"
    lock_trust: str = ""
    induct_in: bool = False
    induct_mix: bool = False
    induct_pos: bool = False
    token_counts: str = ""
    opaque: float = 0.0
    opaque_thr: float = 5.0
    fused_ce: bool = True         # FUSED=ours: fused projection + CE (+mixture) with grads made in forward
    ce_chunk: int = 0             # vocab-chunked CE
    ce_save: bool = False
    short_v: int = 0
    rare_cap: float = 0.3
    reread_anch: float = 0.0      # REREAD_ANCH: only this share of every segment's words, the most surprising ones, re-read
    panic: float = 0.0
    head_dim: int = 64

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)


@dataclass
class OptConfig:
    """InstinctOptB constructor (exp_opt.py:437-439) plus the env switches around it."""
    kind: str = "instinct"        # instinct | experience (the first card optimizer, host-synchronous) | adamw | surprise | muon
    muon_mul: float = 1.0         # MUON_MUL: Muon's learning rate as a multiple of the shared one
    lr: float = 1e-3
    weight_decay: float = 0.1
    cards: int = 4
    beta: float = 0.9
    new_card: float = 0.5
    ema: float = 0.98
    good: float = 0.05
    bad: float = 0.2
    top: float = 0.1
    relax: float = 0.01
    scale: float = 0.2
    lr_peak: Optional[float] = None
    norm: str = "tensor"          # tensor | row | hs | hs<n>
    m_bf16: bool = False
    rel_every: int = 1
    hs_lag: bool = False          # OPT_HS_LAG: one-pass homeostasis with last step's second-axis norm
    sr: bool = False              # stochastic rounding of bf16 stores (BF16_ALL / OPT_SR)
    no_master: bool = False       # BF16_ALL: no fp32 master copies
    offload_m: bool = False       # OPT_OFFLOAD: momentum lives in pinned host memory, on the device only during its update
    vocab_lr_mul: float = 1.0
    sparse_rows: bool = False
    in_backward: bool = True      # stage B: update each weight from its grad-ready hook
    bf16_weights: bool = True     # BF16_W: linear weights live in bf16, exact fp32 copy in the optimizer
    damp: float = 0.0             # >0: per-tensor gradient-surge damping: |g| above damp x its usual norm is clipped
    damp_p: float = 1.0           #     into the momentum and the tensor's step shrinks by (damp x usual / |g|)^damp_p
    damp_beta: float = 0.99       #     EMA of the usual squared norm (per situation card)
    damp_cap: float = 2.0         #     a surge enters that EMA as at most (cap x usual)^2: the brake does not get used to it
    gnorm: bool = False           # every weight's gradient is divided by its own rms before it enters the momentum
    wd_norm: float = 0.0          # >0: decoupled weight decay towards zero for the 1-D norm weights (norm, l_norm, *.n1, *.n2)
    norm_anchor: bool = False     # 1-D norm weights of the light / final blocks are pulled towards 1: w -= lr wd (w - 1)
    lr_mul: tuple = ()            # ((name prefix, multiplier), ...): step multiplier of the weights under a prefix
    stream_proj: bool = False     # light-block matrices: gradient and momentum lose their component along the stream's common vector
    stream_d: int = 0             # width of the stream (0: taken from the matrices)
    m_rate: bool = False          # ... and the common-vector part of their move is rate-limited, the excess banked
    m_rate_kappa: float = 2.0
    m_rate_warm: int = 100
    m_rate_gate: bool = False
    gnorm_rawrel: bool = False    # with gnorm: |g|/|w| (blame, cards) from the raw gradient
    snr_skip: Tuple[str, ...] = ()  # the confidence brake leaves tensors with these name prefixes alone
    snr_only: Tuple[str, ...] = ()  # ... or acts only on these
    safe16: bool = False          # light blocks + output norms: step direction never against the fresh gradient
    safe16_prefix: Tuple[str, ...] = ("light_a.", "light_b.", "final.")
    culprit: str = "abs"          # "abs": the tensors with the largest |g|/|w| are blamed; "ema": the largest against their own mean
    g_max: float = 3.0            # ceiling of a gain
    card_by_kind: bool = False    # the kind of the step (a number given to `prepare`) names the card
    err_step: bool = False        # with damp > 0: every tensor's step x clip(usual |g| / |g| now, 0, err_cap) ("divide by
    err_cap: float = 3.0          #     the sensitivity"); the gradient enters the momentum unclipped
    gearbox: bool = False         # with damp > 0: per-tensor gears (0.25, 0.5, 1, gb_top) shifted one at a time - down when
    gb_down: float = 2.0          #     |g| > gb_down x usual (or when above the limit 1.0 while the loss is worse than
    gb_up: float = 1.3            #     expected), up when |g| < gb_up x usual and the speed has reached the gear; the
    gb_acc: float = 0.05          #     step multiplier moves towards the gear by at most gb_acc per step
    gb_top: float = 1.25
    snr: bool = False             # confidence brake: step x clip(|m_new| / sqrt(EMA |g|^2) / snr_ref, snr_floor, 1) per tensor
    snr_beta: float = 0.95
    snr_ref: float = 1.0
    snr_floor: float = 0.1
    snr_dz: bool = False          #     dead-zone form: brakes only a random walk (see Instinct._snr)
    snr_horizon: float = 250.0
    surge_thr: float = 0.0        # >0: surprise brake: a step much worse than expected (-s > thr) scales lr by (thr/-s)^2


@dataclass
class ParallelConfig:
    world: int = 1
    rank: int = 0
    local_rank: int = 0
    dp: bool = True               # replicate non-expert weights, reduce grads
    ep: bool = True               # shard experts over ranks, all-to-all tokens
    fused: bool = True            # in-kernel peer loads/stores; False = NCCL-only baseline mode
    nvls: bool = True             # multimem paths where available
    wait_ms: float = 2000.0       # bound of every device-side peer wait


@dataclass
class TrainConfig:
    name: str = "Fv2moeK8h8d2048"
    stage: str = "ABX"
    steps: int = 2000
    batch: int = 32
    micro: int = 32
    seq: int = 1024
    lr: float = 3e-4
    read_cost: float = 0.01
    eval_every: int = 100
    warmup: int = 200             # WARMUP
    lr_sched: str = "cosine"      # cosine | wsd
    wsd_frac: float = 0.2
    lr_floor: float = 0.1
    seed: int = 0
    ckpt_dir: str = ""
    ckpt_every: int = 0
    rb_ratio: float = 0.0         # loss-spike rollback guard (0 = off)
    rb_warm: int = 50
    rb_lr: float = 0.5
    nan_guard: bool = True
    watchdog_s: float = 0.0


_TRUE = ("1", "true", "yes", "on")


def _flag(env, name, default=False):
    v = env.get(name)
    if v is None:
        return default
    return v.strip().lower() in _TRUE or (v != "" and v.strip().lower() not in ("0", "false", "no", "off"))


def model_from_env(cfg: ModelConfig, env=None) -> ModelConfig:
    """Apply the reference's environment switches (read in full2.py, full.py and lm.py of the reference) to `cfg`."""
    env = os.environ if env is None else env
    kw = {}
    g = env.get
    if g("ANCHOR_CAP"): kw["cap"] = float(g("ANCHOR_CAP"))
    if g("ANCHOR_FRAC"): kw["frac"] = float(g("ANCHOR_FRAC"))
    if g("CKPT"): kw["ckpt"] = g("CKPT")
    # ACT_CKPT (the reference's per-layer activation checkpointing, fastloop.py:180-262): every layer recomputes in the
    # backward pass.  Its "sel" policy keeps the outputs of library matmuls and recomputes the cheap ops; the layers
    # here run on own autograd functions that already keep exactly what their backward needs, so "sel" is the same as on
    elif g("ACT_CKPT"): kw["ckpt"] = "1"
    if g("NO_MEM"): kw["no_mem"] = True
    if g("NO_REREAD"): kw["no_reread"] = True
    if g("MOE_K"): kw["moe_k"] = int(g("MOE_K"))
    if g("MOE_ACT") == "relu2": kw["moe_act"] = "relu2"
    if g("BF16_EXPERTS") == "1": kw["bf16_experts"] = True
    if g("BANK_Q"): kw["bank_q"] = g("BANK_Q")
    if g("WAVE_WARM"): kw["wave_warm"] = int(g("WAVE_WARM"))
    if g("MOE_CAP_ALIGN"): kw["moe_cap_align"] = int(g("MOE_CAP_ALIGN"))
    # MOE_DISP / MOE_GATHER choose among the reference's dispatch forms; this build has one form (slot table + inverse
    # gather): accepted and ignored.  MOE_GMM (the reference's dropless grouped-GEMM path, full2.py:1048-1100) turns on
    # `moe_dropless`: every expert gets a place for every anchor, so nothing is dropped, and the grouped GEMMs skip the
    # unfilled places through the per-expert fill counts
    if g("MOE_GMM") == "1": kw["moe_dropless"] = True
    if g("MOE_GROUP"): kw["moe_group"] = int(g("MOE_GROUP"))
    if g("LAYER_STATS") == "1": kw["layer_stats"] = True
    if g("HEAVY_ATTN"): kw["heavy_attn"] = True
    if g("HEAVY_ATTN_DETACH"): kw["heavy_attn_detach"] = True
    if g("DRAFT"): kw["n_draft"] = int(g("DRAFT"))
    if g("DRAFT_LOSS"): kw["draft_loss"] = float(g("DRAFT_LOSS"))
    if g("INST_WORD") == "1":
        kw["inst_word"] = True
        for k_ in ("ok", "spread", "target", "spread_w", "cw", "cw_w", "delta"):
            if g("IW_" + k_.upper()): kw["iw_" + k_] = float(g("IW_" + k_.upper()))
        if g("IW_K"): kw["iw_k"] = int(g("IW_K"))
        for k_ in ("rewrite", "random"):
            if g("IW_" + k_.upper()) == "1": kw["iw_" + k_] = True
    if g("NORM_DUMP_PROJ") == "1": kw["norm_dump_proj"] = True
    if g("SAFE_NORM_RATIO"): kw["safe_norm_ratio"] = float(g("SAFE_NORM_RATIO"))
    if g("SAFE_NORM_T0"): kw["safe_norm_t0"] = int(g("SAFE_NORM_T0"))
    if g("HN_GUARD_W"): kw["hn_guard_w"] = float(g("HN_GUARD_W"))
    if g("HN_GUARD_MEAN"): kw["hn_guard_mean"] = float(g("HN_GUARD_MEAN"))
    if g("HN_GUARD_LEN"): kw["hn_guard_len"] = float(g("HN_GUARD_LEN"))
    if g("ATTN_GAIN"): kw["attn_gain"] = float(g("ATTN_GAIN"))
    if g("PREV_IN") == "1": kw["prev_in"] = True
    if g("HEAVY_ROTATE") == "1": kw["heavy_rotate"] = True
    if g("HEAVY_FULL_EVERY"): kw["heavy_full_every"] = int(g("HEAVY_FULL_EVERY"))
    if g("HEAVY_ALL") == "1": kw["heavy_all"] = True
    if g("FISH_N"):
        kw["fish_n"] = int(g("FISH_N"))
        for k_ in ("hf", "kinds", "pool", "c", "eval_c"):
            if g("FISH_" + k_.upper()): kw["fish_" + k_] = int(g("FISH_" + k_.upper()))
        for k_ in ("eval", "center"):
            if g("FISH_" + k_.upper()) == "1": kw["fish_" + k_] = True
    if g("UROBOROS") == "1" or g("HOOP") == "1":
        kw["uroboros"] = True
        for k_, t_ in (("budget", float), ("eat", float), ("w", float), ("thr", float), ("at", str)):
            if g("UROBOROS_" + k_.upper()): kw["uroboros_" + k_] = t_(g("UROBOROS_" + k_.upper()))
        if g("UROBOROS_LEVELS"): kw["uroboros_levels"] = tuple(float(v) for v in g("UROBOROS_LEVELS").split(","))
    if g("ROPE_MEM") == "1":
        kw["rope_mem"], kw["no_mem"] = True, True
        for k_, t_ in (("k", int), ("links", int), ("win", int), ("span_cap", int), ("route", str), ("hier_g", int),
                       ("hier_nb", int), ("hier_bm", int), ("chunk", int), ("layers", int), ("tau0", float),
                       ("frac", float), ("cap", float), ("qfrac", float), ("qtau0", float), ("doc_eos", int),
                       ("pcut", float)):
            if g("ROPE_" + k_.upper()): kw["rope_" + k_] = t_(g("ROPE_" + k_.upper()))
        for k_ in ("share_route", "anchor_top", "key_diag", "route_bf16"):
            if g("ROPE_" + k_.upper()) == "1": kw["rope_" + k_] = True
        if g("ROPE_EXCL_WIN") == "0": kw["rope_excl_win"] = False
        if g("ROPE_RGRAD") == "0": kw["rope_rgrad"] = False
    if g("REMIND_USE_W"): kw["remind_use_w"] = float(g("REMIND_USE_W"))
    if g("REMIND_W"): kw["remind_w"] = float(g("REMIND_W"))
    if g("REMIND_W_SYNTH"): kw["remind_w_synth"] = float(g("REMIND_W_SYNTH"))
    if g("REMIND_N"): kw["remind_q"] = int(g("REMIND_N"))
    if g("REMIND_PER_ROW"): kw["remind_cap"] = int(g("REMIND_PER_ROW")) * int(g("REMIND_N") or 16)
    for k_ in ("mean", "only", "cand", "mask_main", "strict"):
        if g("REMIND_" + k_.upper()) == "1": kw["remind_" + k_] = True
    if g("REMIND_STRICT_W"): kw["remind_strict_w"] = float(g("REMIND_STRICT_W"))
    if g("REMIND_TOK0"): kw["remind_tok0"] = int(g("REMIND_TOK0"))
    if g("BLK"): kw["blk"] = tuple(s for s in g("BLK").split(",") if s)
    if g("LIGHT_FFN"): kw["light_ffn"] = float(g("LIGHT_FFN"))
    if g("LIGHT_MOE"): kw["light_moe"] = g("LIGHT_MOE")
    # ATTN_IMPL (block / block2 window forms of the reference) is accepted and ignored: one windowed attention here
    if g("ROPE_HALF") == "1": kw["rope_half"] = True
    if g("RESID_BF16") == "1": kw["resid_bf16"] = True
    if g("PHRASE_INIT"): kw["phrase_init"] = g("PHRASE_INIT")
    if g("PHRASE_C"): kw["phrase_c"] = float(g("PHRASE_C"))
    if g("SURP_PHRASE"): kw["surp_phrase"] = True
    if g("PHRASE3"): kw["phrase3"] = g("PHRASE3")
    if g("PHR_HASH"): kw["phr_hash"] = True
    if g("PHR_V"): kw["phr_v"] = int(g("PHR_V"))
    if g("PHRASE4"): kw["phrase4"] = g("PHRASE4")
    if g("SKIP"): kw["skip"] = g("SKIP")
    if g("SKIP_G"): kw["skip_g"] = float(g("SKIP_G"))
    if g("TONGUE"): kw["tongue"] = g("TONGUE")
    if g("TONGUE_A"): kw["tongue_a"] = float(g("TONGUE_A"))
    if g("INDUCT"): kw["induct"] = g("INDUCT")
    if g("LOCK_TRUST"): kw["lock_trust"] = g("LOCK_TRUST")
    if g("INDUCT_IN"): kw["induct_in"] = True
    if g("INDUCT_MIX"): kw["induct_mix"] = True
    if g("INDUCT_POS") == "1": kw["induct_pos"] = True
    if g("TOKEN_COUNTS"): kw["token_counts"] = g("TOKEN_COUNTS")
    if g("OPAQUE"): kw["opaque"] = float(g("OPAQUE"))
    if g("OPAQUE_THR"): kw["opaque_thr"] = float(g("OPAQUE_THR"))
    if "FUSED" in env: kw["fused_ce"] = g("FUSED") in ("ours", "liger")
    if g("CE_CHUNK"): kw["ce_chunk"] = int(g("CE_CHUNK"))
    if g("CE_SAVE") == "1": kw["ce_save"] = True
    if g("SHORT_V"): kw["short_v"] = int(g("SHORT_V"))
    if g("RARE_CAP"): kw["rare_cap"] = float(g("RARE_CAP"))
    if g("REREAD_ANCH"): kw["reread_anch"] = float(g("REREAD_ANCH"))
    if g("MEM_LEAN") == "0": kw["memory"] = dataclasses.replace(cfg.memory, lean=False)
    return cfg.replace(**kw)


def opt_from_env(cfg: OptConfig, env=None) -> OptConfig:
    """OPT_KW JSON and the OPT_* / BF16_* switches (fastloop.py:319, exp_opt.py:186, 326)."""
    env = os.environ if env is None else env
    kw = {}
    if env.get("OPT_KW"):
        for k, v in json.loads(env["OPT_KW"]).items():
            if k in OptConfig.__dataclass_fields__:
                kw[k] = v
    if env.get("OPT") == "muon":
        kw["kind"] = "muon"
        kw["muon_mul"] = float(env.get("MUON_MUL", 1))
    if env.get("OPT_HS_LAG") == "1": kw["hs_lag"] = True
    if (env.get("BF16_ALL") == "1" or env.get("OPT_SR") == "1") and env.get("OPT_SR_OFF") != "1": kw["sr"] = True
    if env.get("BF16_ALL") == "1": kw["no_master"] = True
    if env.get("OPT_OFFLOAD") == "1": kw["offload_m"] = True
    if env.get("VOCAB_LR_MUL"): kw["vocab_lr_mul"] = float(env["VOCAB_LR_MUL"])
    if env.get("SPARSE_ROWS"): kw["sparse_rows"] = True
    if env.get("OPT_ALL") == "1": kw["in_backward"] = False
    if "BF16_W" in env: kw["bf16_weights"] = env.get("BF16_W") == "1"
    return dataclasses.replace(cfg, **kw)


def train_from_env(cfg: TrainConfig, env=None) -> TrainConfig:
    env = os.environ if env is None else env
    kw = {}
    if env.get("WARMUP"): kw["warmup"] = int(env["WARMUP"])
    if env.get("LR_SCHED"): kw["lr_sched"] = env["LR_SCHED"]
    if env.get("WSD_FRAC"): kw["wsd_frac"] = float(env["WSD_FRAC"])
    if env.get("LR_FLOOR"): kw["lr_floor"] = float(env["LR_FLOOR"])
    if env.get("CKPT_DIR"): kw["ckpt_dir"] = env["CKPT_DIR"]
    if env.get("CKPT_EVERY"): kw["ckpt_every"] = int(env["CKPT_EVERY"])
    return dataclasses.replace(cfg, **kw)


_SMALL_MEM = dict(fresh=64, dim=128, dim_max=160, write=16, focus=4)


def preset(name: str, vocab: int = 50304, env=None) -> ModelConfig:
    """Model-name grammar of the FullLM2 family (full2.py:2000-2058).

    `Fv2moeK<E>[h<H>][d<D>]` = bank MoE with E experts, H heavy layers (default 14), width D (default 768);
    heads = D // HEAD_DIM (64), LIGHT env = light layers before and after memory (default 2), SEG = segment.
    """
    env = os.environ if env is None else env
    M = lambda **kw: MemoryConfig(**kw)
    if name == "Fv2":
        c = ModelConfig(vocab=vocab)
    elif name == "Fv2_nomem":
        c = ModelConfig(vocab=vocab, ckpt="1", use_memory=False)
    elif name in ("Fv2ck", "Fv2ckg"):
        c = ModelConfig(vocab=vocab, ckpt="1")
    elif name in ("Fv2moe", "Fv2moeB"):
        c = ModelConfig(vocab=vocab, moe="budget" if name == "Fv2moeB" else "fixed")
    elif name in ("Fv2moeW", "Fv2moeWs", "Fv2moeW5", "Fv2moeWsN"):
        c = ModelConfig(vocab=vocab, moe="fixed", wave="still" if name in ("Fv2moeWs", "Fv2moeWsN") else "err",
                        hint_w=0.0 if name == "Fv2moeWsN" else 1.0, err_thr=0.6 if name == "Fv2moeW5" else 0.3)
    elif name in ("Fv3s", "Fv3s_big16"):
        big = name == "Fv3s_big16"
        c = ModelConfig(vocab=vocab, d=256, light_a=1, light_b=1, heavy=2, final=1, heads=4, window=64, seg=32,
                        memory=M(fresh=64 if big else 16, dim=128 if big else 32, dim_max=160 if big else 48,
                                 write=16 if big else 8, focus=4, volume=True))
    elif name.startswith("Fv2moeKs"):
        c = ModelConfig(vocab=vocab, d=256, light_a=1, light_b=1, heavy=3, final=1, heads=4, window=128, seg=64,
                        moe="fixed", n_exp=int(name[8:]), bank=True, memory=M(**_SMALL_MEM))
    elif name.startswith("Fv2moeK"):
        rest, _, dd = name[7:].partition("d")
        e, _, h = rest.partition("h")
        d = int(dd) if dd else 768
        L = int(env.get("LIGHT", 2))
        hd = int(env.get("HEAD_DIM", 64))
        c = ModelConfig(vocab=vocab, d=d, heads=d // hd, head_dim=hd, moe="fixed", n_exp=int(e), bank=True,
                        heavy=int(h) if h else 14, light_a=L, light_b=L, seg=int(env.get("SEG", 512)))
    elif name.startswith("Fv2moeE"):
        e, _, fr = name[7:].partition("f")
        E = int(e)
        c = ModelConfig(vocab=vocab, d=768, heads=12, moe="fixed", n_exp=E,
                        n_frozen=int(E * int(fr) / 100) if fr else 0)
    elif name in ("Fns", "Fns_nomem"):
        c = ModelConfig(vocab=vocab, d=384, light_a=1, light_b=1, heavy=3, final=1, heads=6, window=128, seg=64,
                        ckpt="1", memory=M(**_SMALL_MEM), use_memory=name == "Fns")
    elif name in ("Fn", "Fn_nomem"):
        c = ModelConfig(vocab=vocab, d=512, light_a=2, light_b=2, heavy=4, final=1, heads=8, window=256, seg=128,
                        ckpt="1", memory=M(**_SMALL_MEM), use_memory=name == "Fn")
    elif name == "Fv2s_big16s64":
        c = ModelConfig(vocab=vocab, d=256, light_a=1, light_b=1, heavy=2, final=1, heads=4, window=64, seg=64,
                        memory=M(fresh=64, dim=128, dim_max=160, write=32, focus=4))
    elif name in ("Fv2s_big", "Fv2s_big16"):
        c = ModelConfig(vocab=vocab, d=256, light_a=1, light_b=1, heavy=2, final=1, heads=4, window=64, seg=32,
                        memory=M(fresh=64, dim=128, dim_max=160, write=16 if name == "Fv2s_big16" else 8, focus=4))
    elif name in ("Fv2s", "Fv2s_nomem", "Fv2s_w16"):
        c = ModelConfig(vocab=vocab, d=256, light_a=1, light_b=1, heavy=2, final=1, heads=4, window=64, seg=32,
                        memory=M(fresh=16, dim=32, dim_max=48, write=16 if name == "Fv2s_w16" else 8, focus=4),
                        use_memory=name != "Fv2s_nomem")
    elif name == "tiny":
        # smallest end-to-end slice: d=256, 4 heads, 2+2 light layers window 128, 2 heavy MoE layers of 4 experts
        # (expert hidden 2d -> SwiGLU ffn 1024), top-2 on anchors, memory off
        c = ModelConfig(vocab=vocab, d=256, heads=4, light_a=2, light_b=2, heavy=2, final=0, window=128, seg=64,
                        moe="fixed", n_exp=4, bank=True, no_mem=True)
    elif name == "dense_v2_300m":
        c = ModelConfig(vocab=vocab, d=1024, heads=16, light_a=2, light_b=2, heavy=12, final=0, window=256,
                        memory=M(fresh=64, dim=64, dim_max=96), induct="lock", induct_mix=True)
    elif name == "longctx_1024":
        c = ModelConfig(vocab=vocab, d=1024, heads=16, light_a=4, light_b=4, heavy=6, final=2, window=256,
                        moe="fixed", n_exp=8, bank=True)
    else:
        raise ValueError(f"unknown memarch model name: {name}")
    return model_from_env(c, env)


def published_recipe_env(art_dir: str) -> dict:
    """Environment of the reference's published 2.25B run (scripts/g4_1b_b.py:5-8) with artefact paths under
    `art_dir` (built by memarch_b200.data.phrasebook from the training corpus)."""
    return {
        "FUSED": "ours", "BF16_EXPERTS": "1", "MOE_ACT": "relu2", "LR_SCHED": "wsd", "WSD_FRAC": "0.5",
        "WARMUP": "50",
        "OPT_KW": json.dumps({"norm": "hs", "scale": 0.12, "m_bf16": True, "rel_every": 8}),
        "PHRASE_INIT": os.path.join(art_dir, "bigram.pt"), "PHRASE3": os.path.join(art_dir, "trigram.pt"),
        "SURP_PHRASE": "1", "NO_MEM": "1", "INDUCT": "lock", "LOCK_TRUST": os.path.join(art_dir, "lock_trust.pt"),
        "INDUCT_IN": "1", "INDUCT_MIX": "1", "WAVE_WARM": "1000000",
        "TOKEN_COUNTS": os.path.join(art_dir, "token_counts.npy"),
    }
