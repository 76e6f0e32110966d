"""ReSET: step-aware temperature from token entropy, on the device.

Mirror of reset/reset/logits_processor.py of the reference. Per token with entropy
H_t: T_t = T_low if H_t < tau_t else T_high, with tau_t = tau_0 while the step
entropy H_step is not above the running mean H_bar, and tau_t = H_step otherwise
(reference :1-13). Here the entropy, the per-request bookkeeping, the decision and
the temperature scaling run in ONE kernel launch per step for the whole batch (three
stream-ordered launches for shapes the single launch does not take) with the state
resident on the GPU, so there is no device->host synchronisation per token
(the reference calls ``.item()`` for every request and token, :36).

* :class:`ReSETRequest` - per-request callable ``(output_ids, logits[V]) -> logits``,
  the reference's class of the same name (:62-134).
* :class:`ReSETBatchProcessor` - vLLM v1 batch-level ``LogitsProcessor``: one fused
  step for all requests of the batch.
* ``ReSETAdapter`` - the reference's adapter (:137-155), built on demand because it
  needs vLLM's ``AdapterLogitsProcessor``.
"""

from __future__ import annotations

import ctypes as C
from typing import Iterable, Optional, Sequence

import torch

from .. import _lib, capi

_STATE_BYTES = C.sizeof(_lib.ResetState)
_DECISION_BYTES = C.sizeof(_lib.ResetDecision)


def entropy_of(logits: torch.Tensor) -> torch.Tensor:
    """Shannon entropy (nats) of softmax(logits) with the reference's clamp
    (:32-36). Returns a device tensor ([B] for [B,V] input, scalar for [V]); no
    host synchronisation - call ``.item()`` yourself if a float is wanted."""
    x = logits if logits.dim() == 2 else logits.unsqueeze(0)
    h = capi.entropy(x.float() if x.dtype != torch.float32 else x)
    return h if logits.dim() == 2 else h[0]


def scale_by_temperature(logits: torch.Tensor, temp: float) -> torch.Tensor:
    """``logits / temp``; one-hot at the argmax for ``temp <= 1e-6`` (:22-29)."""
    if temp <= 1e-6:
        out = torch.full_like(logits, float("-inf"))
        out.scatter_(-1, torch.argmax(logits, dim=-1, keepdim=True), 0.0)
        return out
    return logits / temp


def get_newline_token_ids(tokenizer) -> tuple[list[int], list[int]]:
    """Scan the vocabulary once for step-boundary ids (:39-59): ``nl_ids`` decode to
    exactly one newline, ``dnl_ids`` contain a double newline."""
    nl_ids, dnl_ids = [], []
    for tid in range(tokenizer.vocab_size):
        try:
            text = tokenizer.decode([tid], skip_special_tokens=False)
        except Exception:
            continue
        if text == "\n":
            nl_ids.append(tid)
        if "\n\n" in text:
            dnl_ids.append(tid)
    return nl_ids, dnl_ids


def _bitmap(ids: Iterable[int], vocab: int, device) -> Optional[torch.Tensor]:
    """ceil(vocab/32) 32-bit words with bit (id % 32) of word (id // 32) set."""
    ids = sorted({int(i) for i in ids if 0 <= int(i) < vocab})
    if not ids:
        return None
    words = [0] * ((vocab + 31) // 32)
    for i in ids:
        words[i >> 5] |= 1 << (i & 31)
    signed = [w - (1 << 32) if w >= (1 << 31) else w for w in words]
    return torch.tensor(signed, dtype=torch.int32, device=device)


_PARAM_BYTES = C.sizeof(_lib.ResetParams)
_MAX_ID_SETS = 8


class _DeviceReset:
    """Device-side storage shared by the request- and batch-level front ends: one state record,
    one decision record and one hyper-parameter record per slot, and up to ``_MAX_ID_SETS``
    distinct (newline ids, double-newline ids) bitmap pairs that the records refer to."""

    def __init__(self, slots: int, vocab: int, device, pin: bool = False):
        self.device = torch.device(device)
        self.vocab = int(vocab)
        self.slots = int(slots)
        self.words = (self.vocab + 31) // 32
        self.states = torch.zeros(slots * _STATE_BYTES, dtype=torch.uint8, device=self.device)
        self.decisions = torch.zeros(slots * _DECISION_BYTES, dtype=torch.uint8, device=self.device)
        self.workspace = capi.reset_workspace(slots, self.device)
        self.params_host = torch.zeros(slots * _PARAM_BYTES, dtype=torch.uint8, pin_memory=pin)
        self.params_dev = torch.zeros(slots * _PARAM_BYTES, dtype=torch.uint8, device=self.device)
        self.nl_bitmaps = torch.zeros(_MAX_ID_SETS * self.words, dtype=torch.int32, device=self.device)
        self.dnl_bitmaps = torch.zeros(_MAX_ID_SETS * self.words, dtype=torch.int32, device=self.device)
        self._id_sets: dict = {}
        self.slot_record: dict[int, _lib.ResetParams] = {}

    def _id_set(self, nl_ids, dnl_ids) -> int:
        key = (frozenset(int(i) for i in nl_ids), frozenset(int(i) for i in dnl_ids))
        idx = self._id_sets.get(key)
        if idx is None:
            idx = len(self._id_sets)
            if idx >= _MAX_ID_SETS:
                raise ValueError(f"more than {_MAX_ID_SETS} distinct newline-id sets in one processor")
            for store, ids in ((self.nl_bitmaps, key[0]), (self.dnl_bitmaps, key[1])):
                bm = _bitmap(ids, self.vocab, self.device)
                if bm is not None:
                    store[idx * self.words:(idx + 1) * self.words].copy_(bm)
            self._id_sets[key] = idx
        return idx

    @property
    def n_id_sets(self) -> int:
        return len(self._id_sets)

    def set_slot(self, slot: int, t_high: float, t_low: float, tau0: float, window: int,
                 nl_ids: Sequence[int], dnl_ids: Sequence[int]) -> _lib.ResetParams:
        """Start a request in ``slot``: zero its state and write ITS hyper-parameters
        (reference: one ``ReSETRequest`` per request from its own ``extra_args``, :144-155)."""
        if not 1 <= int(window) <= _lib.RESET_MAX_WINDOW:
            raise ValueError(f"window must be in 1..{_lib.RESET_MAX_WINDOW}")
        rec = _lib.ResetParams(float(t_high), float(t_low), float(tau0), int(window),
                               self._id_set(nl_ids, dnl_ids))
        lo, hi = slot * _PARAM_BYTES, (slot + 1) * _PARAM_BYTES
        self.params_host[lo:hi] = torch.frombuffer(bytearray(bytes(rec)), dtype=torch.uint8)
        self.params_dev[lo:hi].copy_(self.params_host[lo:hi], non_blocking=True)
        self.slot_record[slot] = rec
        self.clear_slot(slot)
        return rec

    def move_slot(self, a: int, b: int, swap: bool) -> None:
        """Request in slot ``a`` moves to ``b`` (or the two trade places): state and parameters."""
        for buf, n in ((self.states, _STATE_BYTES), (self.params_dev, _PARAM_BYTES),
                       (self.params_host, _PARAM_BYTES)):
            sa, sb = buf[a * n:(a + 1) * n], buf[b * n:(b + 1) * n]
            if swap:
                tmp = sb.clone()
                sb.copy_(sa)
                sa.copy_(tmp)
            else:
                sb.copy_(sa)
        ra, rb = self.slot_record.pop(a, None), self.slot_record.pop(b, None)
        if ra is not None:
            self.slot_record[b] = ra
        if swap and rb is not None:
            self.slot_record[a] = rb

    def clear_slot(self, slot: int) -> None:
        self.states[slot * _STATE_BYTES:(slot + 1) * _STATE_BYTES].zero_()


class ReSETRequest:
    """Per-request policy with the reference's constructor and call signature
    (:62-134): ``req(output_ids, logits[V]) -> logits[V]``. The returned tensor is a
    new tensor (the reference does not modify its input either)."""

    def __init__(self, t_high, t_low, tau_raw, window, nl_ids, dnl_ids):
        self.t_high, self.t_low, self.tau_raw = float(t_high), float(t_low), float(tau_raw)
        self.window = int(window)
        self.nl_ids = frozenset(int(x) for x in nl_ids)
        self.dnl_ids = frozenset(int(x) for x in dnl_ids)
        self._dev: Optional[_DeviceReset] = None
        self._last = None

    def __call__(self, output_ids, logits: torch.Tensor) -> torch.Tensor:
        if self._dev is None:
            self._dev = _DeviceReset(1, logits.shape[-1], logits.device)
            self._dev.set_slot(0, self.t_high, self.t_low, self.tau_raw, self.window, self.nl_ids, self.dnl_ids)
            self._last = torch.empty((1, 2), dtype=torch.int32, device=logits.device)
        n = len(output_ids)
        host = torch.tensor([[output_ids[-2] if n >= 2 else -1, output_ids[-1] if n >= 1 else -1]],
                            dtype=torch.int32)
        self._last.copy_(host, non_blocking=True)
        out = logits.to(torch.float32, copy=True).unsqueeze(0)
        d = self._dev
        capi.reset_step_per_request(out, d.states, d.params_dev, last_ids=self._last,
                                    nl_bitmaps=d.nl_bitmaps, dnl_bitmaps=d.dnl_bitmaps, n_id_sets=d.n_id_sets,
                                    decisions=d.decisions, workspace=d.workspace)
        return out[0].to(logits.dtype)

    def last_decision(self) -> dict:
        """(entropy, h_step, h_bar, temp, boundary, high_step) of the latest call;
        synchronises - diagnostics only."""
        raw = self._dev.decisions[:_DECISION_BYTES].cpu().numpy().tobytes()
        d = _lib.ResetDecision.from_buffer_copy(raw)
        return {f: getattr(d, f) for f, _ in _lib.ResetDecision._fields_}


class ReSETBatchProcessor:
    """vLLM v1 ``LogitsProcessor`` interface (``__init__(vllm_config, device,
    is_pin_memory)``, ``is_argmax_invariant``, ``update_state``, ``apply``) doing one
    fused ReSET step for the whole batch. Requests opt in through
    ``SamplingParams.extra_args`` with the reference's keys (:144-155): ``reset``,
    ``t_high``, ``t_low``, ``tau_0``, ``window``, ``reset_nl_ids``, ``reset_dnl_ids``.
    Every request keeps its OWN values, as in the reference: they are written into the
    request's slot on the device when the request is admitted, and the kernel reads the
    record of each row's slot."""

    def __init__(self, vllm_config=None, device="cuda", is_pin_memory: bool = False,
                 max_num_reqs: Optional[int] = None, vocab_size: Optional[int] = None):
        self.device = torch.device(device)
        self.pin = bool(is_pin_memory)
        if max_num_reqs is None:
            max_num_reqs = vllm_config.scheduler_config.max_num_seqs
        if vocab_size is None:
            vocab_size = vllm_config.model_config.get_vocab_size()
        self.max_reqs, self.vocab = int(max_num_reqs), int(vocab_size)
        self._dev: Optional[_DeviceReset] = None
        self._outputs: dict[int, list[int]] = {}       # batch index -> live output id list
        self._slots_host = torch.full((self.max_reqs,), -1, dtype=torch.int32, pin_memory=self.pin)
        self._last_host = torch.full((self.max_reqs, 2), -1, dtype=torch.int32, pin_memory=self.pin)
        self._slots_dev = torch.full((self.max_reqs,), -1, dtype=torch.int32, device=self.device)
        self._last_dev = torch.full((self.max_reqs, 2), -1, dtype=torch.int32, device=self.device)
        # host-visible time-out word (no synchronisation to read it); looked at every few steps
        self._mirror = None
        self._steps = 0
        self.check_every = 16

    def is_argmax_invariant(self) -> bool:
        return False

    def _admit(self, idx: int, ea: dict) -> None:
        if self._dev is None:
            self._dev = _DeviceReset(self.max_reqs, self.vocab, self.device, pin=self.pin)
        self._dev.set_slot(idx, float(ea["t_high"]), float(ea["t_low"]), float(ea.get("tau_0", 0.6349)),
                           int(ea.get("window", 32)), ea.get("reset_nl_ids", []), ea.get("reset_dnl_ids", []))

    def update_state(self, batch_update) -> None:
        if batch_update is not None:
            for idx in batch_update.removed:
                self._outputs.pop(idx, None)
                self._slots_host[idx] = -1
            for idx, params, _prompt, out_ids in batch_update.added:
                ea = getattr(params, "extra_args", None) or {}
                if ea.get("reset"):
                    self._admit(idx, ea)
                    self._outputs[idx] = out_ids
                    self._slots_host[idx] = idx
                else:
                    self._outputs.pop(idx, None)
                    self._slots_host[idx] = -1
            for a, b, direction in batch_update.moved:
                swap = getattr(direction, "name", str(direction)) == "SWAP"
                self._move(a, b, swap)
            self._slots_dev.copy_(self._slots_host, non_blocking=True)
        for idx, ids in self._outputs.items():
            n = len(ids)
            self._last_host[idx, 0] = ids[-2] if n >= 2 else -1
            self._last_host[idx, 1] = ids[-1] if n >= 1 else -1
        if self._outputs:
            self._last_dev.copy_(self._last_host, non_blocking=True)

    def _move(self, a: int, b: int, swap: bool) -> None:
        if self._dev is not None:
            self._dev.move_slot(a, b, swap)
        oa, ob = self._outputs.pop(a, None), self._outputs.pop(b, None)
        if oa is not None:
            self._outputs[b] = oa
        if swap and ob is not None:
            self._outputs[a] = ob
        act_a, act_b = int(self._slots_host[a]) >= 0, int(self._slots_host[b]) >= 0
        self._slots_host[b] = b if act_a else -1
        self._slots_host[a] = (a if act_b else -1) if swap else -1

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        if self._dev is None or not self._outputs:
            return logits
        B = logits.shape[0]
        d = self._dev
        work = logits if logits.dtype == torch.float32 else logits.float()
        capi.reset_step_per_request(work, d.states, d.params_dev, state_slots=self._slots_dev[:B],
                                    last_ids=self._last_dev[:B], nl_bitmaps=d.nl_bitmaps,
                                    dnl_bitmaps=d.dnl_bitmaps, n_id_sets=d.n_id_sets,
                                    decisions=d.decisions, workspace=d.workspace)
        if work is not logits:
            logits.copy_(work)
        self._steps += 1
        if self.check_every and self._steps % self.check_every == 0:
            self.raise_on_device_timeout()
        return logits

    def raise_on_device_timeout(self) -> None:
        """Reads the pinned-host twin of the kernels' time-out flags (no device synchronisation).
        A non-zero word means a bounded wait inside an earlier launch gave up: that step's logits
        are undefined and the processor's scratch is mid-exchange, so it is zeroed and the error
        is raised instead of serving wrong temperatures silently."""
        if self._mirror is None:
            with torch.cuda.device(self.device):
                self._mirror = _lib.status_mirror()
        code = int(self._mirror[0])
        if code != 0:
            self._mirror[0] = 0
            if self._dev is not None:
                self._dev.workspace.zero_()
            raise RuntimeError(f"nvfp4r: a device-side wait timed out (kernel family {code}); "
                               "the logits of that step are undefined")


_BATCH_CLASS = None


def make_batch_processor_class():
    """:class:`ReSETBatchProcessor` as vLLM wants it: ``LLM(logits_processors=[cls])`` only
    accepts subclasses of ``vllm.v1.sample.logits_processor.LogitsProcessor``. The subclass is
    built on first use (importing vLLM takes seconds and the kernels do not need it) and has the
    same name and constructor; without vLLM the plain class is returned."""
    global _BATCH_CLASS
    if _BATCH_CLASS is None:
        try:
            from vllm.v1.sample.logits_processor import LogitsProcessor
        except ImportError:
            _BATCH_CLASS = ReSETBatchProcessor
        else:
            _BATCH_CLASS = type("ReSETBatchProcessor", (ReSETBatchProcessor, LogitsProcessor),
                                {"__doc__": ReSETBatchProcessor.__doc__, "__module__": __name__})
    return _BATCH_CLASS


def make_adapter_class():
    """The reference's ``ReSETAdapter`` (:137-155): a vLLM ``AdapterLogitsProcessor``
    producing one :class:`ReSETRequest` per opted-in request."""
    from vllm.v1.sample.logits_processor import AdapterLogitsProcessor

    class ReSETAdapter(AdapterLogitsProcessor):
        def is_argmax_invariant(self) -> bool:
            return False

        def new_req_logits_processor(self, params):
            ea = getattr(params, "extra_args", None) or {}
            if not ea.get("reset"):
                return None
            return ReSETRequest(t_high=float(ea["t_high"]), t_low=float(ea["t_low"]),
                                tau_raw=float(ea.get("tau_0", 0.6349)),
                                window=int(ea.get("window", 32)),
                                nl_ids=ea.get("reset_nl_ids", []), dnl_ids=ea.get("reset_dnl_ids", []))

    return ReSETAdapter
