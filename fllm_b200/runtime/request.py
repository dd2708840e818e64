"""Request-side data: the one sampling contract shared by every API dialect
(rust/engine/src/sampling.rs:6-49, rust/engine/src/parameters.rs:1) and the
per-request state tracked by the scheduler."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    seed: Optional[int] = None
    max_tokens: int = 256
    min_tokens: int = 0
    ignore_eos: bool = False
    stop_token_ids: Sequence[int] = ()
    stop: Sequence[str] = ()
    logit_bias: Optional[Dict[int, float]] = None
    allowed_token_ids: Optional[Sequence[int]] = None
    bad_words_ids: Optional[Sequence[int]] = None
    bad_words: Optional[Sequence[Sequence[int]]] = None    # banned token sequences (the last token is banned after the others)
    typical_p: float = 1.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_sequence_breakers: Sequence[int] = ()
    dry_penalty_last_n: int = 1024
    mirostat_mode: int = 0               # 0 off; 1 = Mirostat (Zipf top-k cut); 2 = Mirostat 2.0 (surprise cut)
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    logprobs: bool = False
    top_logprobs: int = 0
    n: int = 1
    priority: int = 0
    timeout_s: Optional[float] = None
    cache_salt: str = ""
    speculative: bool = True
    embed: bool = False                  # return the final-norm hidden state of the last prompt token (embeddings API)
    guided: Optional[object] = None      # runtime.grammar.GuidedJson: per-step allowed-token mask + advance()
    guided_spec: Optional[dict] = None   # the request fields `guided` was built from (travels to the other ranks)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def needs_full_sampler(self) -> bool:
        return (not self.greedy or self.repetition_penalty != 1.0 or self.presence_penalty != 0.0
                or self.frequency_penalty != 0.0 or bool(self.logit_bias)
                or self.allowed_token_ids is not None or bool(self.bad_words_ids) or self.logprobs
                or self.guided is not None or self.needs_host_processors)

    @property
    def spec_mode(self) -> Optional[str]:
        """How drafts of this request are verified: "greedy" (chain match on the argmax ids), "sampled" (the
        exact accept / residual rule on the temperature-scaled distributions; needs the plain distribution, so
        no truncation, penalty, bias, mask or host processor), or None (not speculated)."""
        if not self.speculative:
            return None
        if not self.needs_full_sampler:
            return "greedy"
        plain = (self.top_k == 0 and self.top_p >= 1.0 and self.min_p <= 0.0 and self.repetition_penalty == 1.0
                 and self.presence_penalty == 0.0 and self.frequency_penalty == 0.0 and not self.logit_bias
                 and self.allowed_token_ids is None and not self.bad_words_ids and not self.logprobs
                 and self.guided is None and not self.needs_host_processors)
        return "sampled" if (plain and self.temperature > 0.0) else None

    @property
    def needs_host_processors(self) -> bool:
        return (self.typical_p < 1.0 or self.dry_multiplier > 0.0 or self.mirostat_mode != 0 or bool(self.bad_words))

    def validate(self, vocab_size: int) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0 <= self.min_p <= 1:
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.n != 1:
            raise ValueError("n > 1 is served by submitting n requests")
        if not 0 < self.typical_p <= 1:
            raise ValueError("typical_p must be in (0, 1]")
        if self.dry_multiplier < 0 or self.dry_base < 1 or self.dry_allowed_length < 1:
            raise ValueError("DRY needs multiplier >= 0, base >= 1, allowed_length >= 1")
        if self.mirostat_mode not in (0, 1, 2) or self.mirostat_tau <= 0 or self.mirostat_eta <= 0:
            raise ValueError("mirostat: mode 0, 1 or 2 with tau > 0 and eta > 0")
        if self.mirostat_mode:
            self.speculative = False         # the controller's state moves one sampled token at a time
        if not 0 <= self.top_logprobs <= 20:
            raise ValueError("top_logprobs must be in [0, 20]")
        if self.logprobs:
            self.speculative = False         # one sampled row per emitted token keeps the log-probability lists aligned
        for t in list(self.stop_token_ids) + list((self.logit_bias or {}).keys()):
            if not 0 <= int(t) < vocab_size:
                raise ValueError(f"token id {t} outside the vocabulary")


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"
    ABORTED = "aborted"


@dataclass
class Request:
    request_id: str
    seq_id: int
    prompt: List[int]
    params: SamplingParams
    arrival: float = field(default_factory=time.monotonic)
    status: RequestStatus = RequestStatus.WAITING
    output: List[int] = field(default_factory=list)
    num_computed: int = 0            # tokens (prompt + output) whose KV is stored
    num_cached: int = 0              # prompt tokens served from the prefix cache
    finish_reason: Optional[str] = None
    first_token_time: Optional[float] = None
    last_token_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    preemptions: int = 0
    draft: List[int] = field(default_factory=list)   # proposed tokens awaiting verification
    draft_logits: Optional[object] = None            # [len(draft), vocab] device tensor when the drafts were sampled
    logprobs: List[float] = field(default_factory=list)
    top_logprobs: List[list] = field(default_factory=list)   # per output token: [(token id, log-probability), ...]
    swapped: bool = False            # preempted with its KV parked in host memory
    mirostat: Optional[object] = None  # runtime.logits_processors.Mirostat, created on first use

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        """Tokens that still have to be fed to the model before the next one can be sampled."""
        return self.num_tokens - self.num_computed

    @property
    def is_decode(self) -> bool:
        return self.remaining == 1 and bool(self.output)

    @property
    def finished(self) -> bool:
        return self.status in (RequestStatus.FINISHED, RequestStatus.ABORTED)

    def deadline_passed(self, now: float) -> bool:
        return self.params.timeout_s is not None and now - self.arrival > self.params.timeout_s


@dataclass
class TokenEvent:
    request_id: str
    token_ids: List[int]
    finished: bool = False
    finish_reason: Optional[str] = None
    logprobs: Optional[List[float]] = None
    error: Optional[str] = None
    embedding: Optional[List[float]] = None
    top_logprobs: Optional[List[list]] = None
