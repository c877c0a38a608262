"""Raise the open-file limit: a peer holds many sockets (reference: hivemind/utils/limits.py:6-17)."""
from hivemind_b200.utils.logging import get_logger

logger = get_logger(__name__)


def increase_file_limit(new_soft: int = 2 ** 15, new_hard: int = 2 ** 15) -> None:
    try:
        import resource

        soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
        target_hard = max(hard, new_hard) if hard != resource.RLIM_INFINITY else hard
        target_soft = max(soft, new_soft)
        if target_hard != resource.RLIM_INFINITY:
            target_soft = min(target_soft, target_hard)
        resource.setrlimit(resource.RLIMIT_NOFILE, (target_soft, target_hard))
    except Exception as e:
        logger.warning(f"could not raise the open-file limit: {e!r}")
