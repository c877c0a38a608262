"""``StepControl``: the handle a caller gets for one averaging step.

It is a future of the step's result plus live controls (reference: hivemind/averaging/control.py:14-165):
``scheduled_time`` and ``weight`` may be changed until the all-reduce begins, ``allow_allreduce()`` releases a step
that was created with ``require_trigger=True``, ``stage`` tells how far the step has come, ``cancel()`` aborts it.
The reference keeps these fields in shared memory because its averager is another process; here the averager is a
thread of the same process, so plain attributes guarded by a lock are enough.
"""
from __future__ import annotations

import threading
from enum import Enum
from typing import Optional

from hivemind_b200.utils import DHTExpiration, MPFuture, get_dht_time, get_logger

logger = get_logger(__name__)


class AveragingStage(Enum):
    IDLE = 0  # still initializing
    LOOKING_FOR_GROUP = 1  # running decentralized matchmaking, can't run allreduce yet
    AWAITING_TRIGGER = 2  # waiting for user to set the trigger that allows running allreduce
    RUNNING_ALLREDUCE = 3  # exchanging tensors with groupmates
    FINISHED = 4  # either done or failed with exception


class StepControl(MPFuture):
    """
    :param scheduled_time: estimated time when averaging should begin; matchmaking aims for it
    :param deadline: if averaging is still in progress at this time, it is cancelled
    :param allow_retries: if matchmaking or all-reduce fails, retry until the deadline
    :param weight: this peer's weight in the average
    :param data_for_gather: opaque blob sent to every groupmate
    """

    def __init__(self, scheduled_time: DHTExpiration, deadline: float, allow_retries: bool, weight: float,
                 data_for_gather: bytes):
        super().__init__()
        self._data_for_gather, self._deadline, self._allow_retries = data_for_gather, deadline, allow_retries
        self._trigger: Optional[MPFuture] = None
        self._cancel: Optional[MPFuture] = None
        self._fields_lock = threading.Lock()
        self._scheduled_time = float(scheduled_time)
        self._weight = float(weight)
        self._stage = AveragingStage.IDLE
        self._began_allreduce = False

    def attach(self, trigger: MPFuture, cancel: MPFuture) -> None:
        assert self._trigger is None and self._cancel is None, "futures are already attached"
        self._trigger, self._cancel = trigger, cancel

    def allow_allreduce(self) -> None:
        """Let a step that requires a trigger proceed to all-reduce as soon as its group is assembled."""
        assert self._trigger is not None, "StepControl does not have an attached trigger"
        if self._trigger.done():
            logger.warning("trigger is already set")
        else:
            self._trigger.set_result(None)

    async def wait_for_trigger(self) -> None:
        assert self._trigger is not None, "StepControl does not have an attached trigger"
        await self._trigger

    @property
    def triggered(self) -> bool:
        assert self._trigger is not None, "StepControl does not have an attached trigger"
        return self._trigger.done()

    @property
    def scheduled_time(self) -> DHTExpiration:
        with self._fields_lock:
            return self._scheduled_time

    @scheduled_time.setter
    def scheduled_time(self, scheduled_time: DHTExpiration) -> None:
        if self.began_allreduce:
            logger.warning("changing scheduled time has no effect after all-reduce has already started")
        if scheduled_time >= self.deadline:
            logger.warning("changing scheduled time to after deadline, averaging will likely fail due to timeout")
        with self._fields_lock:
            self._scheduled_time = float(scheduled_time)

    @property
    def weight(self) -> float:
        with self._fields_lock:
            return self._weight

    @weight.setter
    def weight(self, weight: float) -> None:
        assert weight >= 0 and weight == weight and weight != float("inf"), "weight must be a finite non-negative number"
        if self.began_allreduce:
            logger.warning("changing weights has no effect after all-reduce has already started")
        with self._fields_lock:
            self._weight = float(weight)

    @property
    def stage(self) -> AveragingStage:
        with self._fields_lock:
            return self._stage

    @stage.setter
    def stage(self, stage: AveragingStage) -> None:
        with self._fields_lock:
            if stage == AveragingStage.RUNNING_ALLREDUCE:
                self._began_allreduce = True
            self._stage = stage

    @property
    def began_allreduce(self) -> bool:
        with self._fields_lock:
            return self._began_allreduce

    @property
    def data_for_gather(self) -> bytes:
        return self._data_for_gather

    @property
    def deadline(self) -> DHTExpiration:
        return self._deadline

    def get_timeout(self) -> Optional[DHTExpiration]:
        return max(0.0, self.deadline - get_dht_time())

    @property
    def allow_retries(self) -> bool:
        return self._allow_retries

    def cancel(self) -> bool:
        if self._trigger is not None:
            self._trigger.cancel()
        if self._cancel is not None and not self._cancel.done():
            self._cancel.set_result(None)
        return super().cancel()

    async def wait_for_cancel(self) -> None:
        """Resolves when the user cancels the step."""
        await self._cancel
