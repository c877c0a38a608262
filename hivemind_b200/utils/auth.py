"""Optional authorization for moderated swarms.

Protocol (the one of hivemind/utils/auth.py:33-211, so that the same ``auth.proto`` messages work): an authority
issues short-lived access tokens that bind a username to a peer's RSA public key. A request carries the caller's
token, the current time and a fresh nonce and is signed with the caller's key (optionally naming the key of the
service it is meant for); the service checks the token, the signature, the clock skew and that the nonce has not been
seen, then signs its response together with the request's nonce. ``AuthRPCWrapper`` applies the caller side to a
stub or the service side to a servicer; with ``authorizer=None`` it changes nothing.
"""
from __future__ import annotations

import functools
import inspect
import secrets
import threading
import asyncio
from abc import ABC, abstractmethod
from datetime import timedelta
from enum import Enum
from typing import Optional

from hivemind_b200.proto.auth_pb2 import AccessToken, RequestAuthInfo, ResponseAuthInfo
from hivemind_b200.utils.crypto import RSAPrivateKey, RSAPublicKey
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.timed_storage import TimedStorage, get_dht_time

logger = get_logger(__name__)


class AuthorizedRequestBase:
    """Any protobuf message with a field ``auth`` of type ``RequestAuthInfo``."""

    auth: RequestAuthInfo


class AuthorizedResponseBase:
    """Any protobuf message with a field ``auth`` of type ``ResponseAuthInfo``."""

    auth: ResponseAuthInfo


class AuthorizerBase(ABC):
    """The four hooks of an authorization scheme: caller signs / service checks, service signs / caller checks."""

    @abstractmethod
    async def sign_request(self, request: AuthorizedRequestBase, service_public_key: Optional[RSAPublicKey]) -> None:
        ...

    @abstractmethod
    async def validate_request(self, request: AuthorizedRequestBase) -> bool:
        ...

    @abstractmethod
    async def sign_response(self, response: AuthorizedResponseBase, request: AuthorizedRequestBase) -> None:
        ...

    @abstractmethod
    async def validate_response(self, response: AuthorizedResponseBase, request: AuthorizedRequestBase) -> bool:
        ...


def _attach_signature(message, key: RSAPrivateKey) -> None:
    """Sign ``message`` with its ``auth.signature`` field empty and store the signature there."""
    assert message.auth.signature == b"", "the message is already signed"
    message.auth.signature = key.sign(message.SerializeToString())


def _signature_is_valid(message, key: RSAPublicKey) -> bool:
    """Check ``auth.signature`` against the message with that field blanked (the field stays blank afterwards)."""
    signature, message.auth.signature = message.auth.signature, b""
    return key.verify(message.SerializeToString(), signature)


class _ReplayGuard:
    """Rejects requests whose clock is too far off or whose nonce was already used inside the acceptance window."""

    def __init__(self, max_skew: timedelta):
        self.max_skew_seconds = max_skew.total_seconds()
        self._seen = TimedStorage()
        self._lock = threading.Lock()

    def admit(self, sent_at: float, nonce: bytes) -> bool:
        with self._lock:
            now = get_dht_time()
            if abs(sent_at - now) > self.max_skew_seconds:
                logger.debug("clocks are not synchronized or a previous request is replayed again")
                return False
            if nonce in self._seen:
                logger.debug("previous request is replayed again")
                return False
            self._seen.store(nonce, None, now + 3 * self.max_skew_seconds)
            return True


class TokenAuthorizerBase(AuthorizerBase):
    """
    Token-based scheme; subclasses say how a token is obtained (``get_token``), whether one is acceptable
    (``is_token_valid``) and when the local one should be renewed (``does_token_need_refreshing``).
    """

    _MAX_CLIENT_SERVICER_TIME_DIFF = timedelta(minutes=1)

    def __init__(self, local_private_key: Optional[RSAPrivateKey] = None):
        self._local_private_key = local_private_key if local_private_key is not None else RSAPrivateKey.process_wide()
        self._local_public_key = self._local_private_key.get_public_key()
        self._local_access_token: Optional[AccessToken] = None
        self._refresh_lock = asyncio.Lock()
        self._replay_guard = _ReplayGuard(self._MAX_CLIENT_SERVICER_TIME_DIFF)

    @property
    def local_public_key(self) -> RSAPublicKey:
        return self._local_public_key

    @abstractmethod
    async def get_token(self) -> AccessToken:
        ...

    @abstractmethod
    def is_token_valid(self, access_token: AccessToken) -> bool:
        ...

    @abstractmethod
    def does_token_need_refreshing(self, access_token: AccessToken) -> bool:
        ...

    def _token_is_stale(self) -> bool:
        return self._local_access_token is None or self.does_token_need_refreshing(self._local_access_token)

    async def refresh_token_if_needed(self) -> None:
        if not self._token_is_stale():
            return
        async with self._refresh_lock:
            if self._token_is_stale():  # somebody else may have refreshed it while we waited for the lock
                token = await self.get_token()
                assert self.is_token_valid(token), "the authority issued a token that this authorizer rejects"
                self._local_access_token = token

    # ---- caller side -------------------------------------------------------------------------------------
    async def sign_request(self, request: AuthorizedRequestBase, service_public_key: Optional[RSAPublicKey]) -> None:
        await self.refresh_token_if_needed()
        info = request.auth
        info.client_access_token.CopyFrom(self._local_access_token)
        info.time, info.nonce = get_dht_time(), secrets.token_bytes(8)
        if service_public_key is not None:
            info.service_public_key = service_public_key.to_bytes()
        _attach_signature(request, self._local_private_key)

    async def validate_response(self, response: AuthorizedResponseBase, request: AuthorizedRequestBase) -> bool:
        await self.refresh_token_if_needed()
        token = response.auth.service_access_token
        if not self.is_token_valid(token):
            logger.debug("service failed to prove that it (still) has access to the network")
            return False
        if not _signature_is_valid(response, RSAPublicKey.from_bytes(token.public_key)):
            logger.debug("response has invalid signature")
            return False
        if response.auth.nonce != request.auth.nonce:
            logger.debug("response is generated for another request")
            return False
        return True

    # ---- service side ------------------------------------------------------------------------------------
    async def validate_request(self, request: AuthorizedRequestBase) -> bool:
        await self.refresh_token_if_needed()
        info = request.auth
        if not self.is_token_valid(info.client_access_token):
            logger.debug("client failed to prove that it (still) has access to the network")
            return False
        if not _signature_is_valid(request, RSAPublicKey.from_bytes(info.client_access_token.public_key)):
            logger.debug("request has invalid signature")
            return False
        if info.service_public_key and info.service_public_key != self._local_public_key.to_bytes():
            logger.debug("request is generated for a peer with another public key")
            return False
        return self._replay_guard.admit(info.time, info.nonce)

    async def sign_response(self, response: AuthorizedResponseBase, request: AuthorizedRequestBase) -> None:
        await self.refresh_token_if_needed()
        response.auth.service_access_token.CopyFrom(self._local_access_token)
        response.auth.nonce = request.auth.nonce
        _attach_signature(response, self._local_private_key)


class AuthRole(Enum):
    CLIENT = 0
    SERVICER = 1


class AuthRPCWrapper:
    """
    Wraps a stub (``AuthRole.CLIENT``: sign requests, check responses) or a servicer (``AuthRole.SERVICER``: check
    requests, sign responses). Only attributes whose names start with ``rpc_`` are intercepted. A request that fails
    validation gets no answer (``None``, or an empty stream).
    """

    def __init__(self, stub, role: AuthRole, authorizer: Optional[AuthorizerBase],
                 service_public_key: Optional[RSAPublicKey] = None):
        self._stub, self._role, self._authorizer = stub, role, authorizer
        self._service_public_key = service_public_key

    def __getattribute__(self, name: str):
        plain = object.__getattribute__
        if not name.startswith("rpc_"):
            return plain(self, name)
        method = getattr(plain(self, "_stub"), name)
        authorizer = plain(self, "_authorizer")
        if authorizer is None:
            return method
        serving = plain(self, "_role") == AuthRole.SERVICER
        target_key = plain(self, "_service_public_key")

        if inspect.isasyncgenfunction(method):
            @functools.wraps(method)
            async def guarded_stream(request, *args, **kwargs):
                if serving and not await authorizer.validate_request(request):
                    return
                async for item in method(request, *args, **kwargs):
                    if serving:
                        await authorizer.sign_response(item, request)
                    yield item

            return guarded_stream

        @functools.wraps(method)
        async def guarded_call(request: AuthorizedRequestBase, *args, **kwargs):
            if serving:
                if not await authorizer.validate_request(request):
                    return None
                response = await method(request, *args, **kwargs)
                await authorizer.sign_response(response, request)
                return response
            await authorizer.sign_request(request, target_key)
            response = await method(request, *args, **kwargs)
            if response is None:  # the service refused to answer
                return None
            return response if await authorizer.validate_response(response, request) else None

        return guarded_call
