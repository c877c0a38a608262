"""Decentralized averaging: matchmaking through the DHT and butterfly all-reduce inside the matched group."""
from hivemind_b200.averaging.allreduce import AllReduceRunner, AveragingMode
from hivemind_b200.averaging.averager import DecentralizedAverager
from hivemind_b200.averaging.control import AveragingStage, StepControl
from hivemind_b200.averaging.partition import AllreduceException, BannedException
