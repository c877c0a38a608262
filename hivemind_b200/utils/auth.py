"""Optional authorization for moderated swarms (reference: hivemind/utils/auth.py:33-211).

An authority signs short-lived access tokens that bind a username to a peer's RSA public key. Every request carries
the client's token, a timestamp and a nonce, signed with the client's key; every response echoes the nonce and is
signed by the service. ``AuthRPCWrapper`` applies this to a stub (client role) or a servicer (servicer role); with
``authorizer=None`` it is a transparent pass-through.
"""
from __future__ import annotations

import asyncio
import functools
import inspect
import secrets
import threading
import time
from abc import ABC, abstractmethod
from datetime import datetime, timedelta, timezone
from enum import Enum
from typing import Optional

from hivemind_b200.proto.auth_pb2 import AccessToken, RequestAuthInfo, ResponseAuthInfo
from hivemind_b200.utils.crypto import RSAPrivateKey, RSAPublicKey
from hivemind_b200.utils.logging import get_logger
from hivemind_b200.utils.timed_storage import TimedStorage, get_dht_time

logger = get_logger(__name__)


class AuthorizedRequestBase:
    """Interface of protobufs that have an ``auth: RequestAuthInfo`` field."""

    auth: RequestAuthInfo


class AuthorizedResponseBase:
    """Interface of protobufs that have an ``auth: ResponseAuthInfo`` field."""

    auth: ResponseAuthInfo


class AuthorizerBase(ABC):
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


class TokenAuthorizerBase(AuthorizerBase):
    """Authorizer based on access tokens issued by an authority; subclasses implement token acquisition and checks."""

    _MAX_CLIENT_SERVICER_TIME_DIFF = timedelta(minutes=1)

    def __init__(self, local_private_key: Optional[RSAPrivateKey] = None):
        if local_private_key is None:
            local_private_key = RSAPrivateKey.process_wide()
        self._local_private_key = local_private_key
        self._local_public_key = local_private_key.get_public_key()
        self._local_access_token: Optional[AccessToken] = None
        self._refresh_lock = asyncio.Lock()
        self._recent_nonces = TimedStorage()
        self._nonce_lock = threading.Lock()

    @abstractmethod
    async def get_token(self) -> AccessToken:
        ...

    @abstractmethod
    def is_token_valid(self, access_token: AccessToken) -> bool:
        ...

    @abstractmethod
    def does_token_need_refreshing(self, access_token: AccessToken) -> bool:
        ...

    async def refresh_token_if_needed(self) -> None:
        if self._local_access_token is None or self.does_token_need_refreshing(self._local_access_token):
            async with self._refresh_lock:
                if self._local_access_token is None or self.does_token_need_refreshing(self._local_access_token):
                    self._local_access_token = await self.get_token()
                    assert self.is_token_valid(self._local_access_token)

    @property
    def local_public_key(self) -> RSAPublicKey:
        return self._local_public_key

    async def sign_request(self, request: AuthorizedRequestBase, service_public_key: Optional[RSAPublicKey]) -> None:
        await self.refresh_token_if_needed()
        auth = request.auth
        auth.client_access_token.CopyFrom(self._local_access_token)
        if service_public_key is not None:
            auth.service_public_key = service_public_key.to_bytes()
        auth.time = get_dht_time()
        auth.nonce = secrets.token_bytes(8)
        assert auth.signature == b""
        auth.signature = self._local_private_key.sign(request.SerializeToString())

    async def validate_request(self, request: AuthorizedRequestBase) -> bool:
        await self.refresh_token_if_needed()
        auth = request.auth
        if not self.is_token_valid(auth.client_access_token):
            logger.debug("client failed to prove that it (still) has access to the network")
            return False
        client_public_key = RSAPublicKey.from_bytes(auth.client_access_token.public_key)
        signature = auth.signature
        auth.signature = b""
        if not client_public_key.verify(request.SerializeToString(), signature):
            logger.debug("request has invalid signature")
            return False
        if auth.service_public_key and auth.service_public_key != self._local_public_key.to_bytes():
            logger.debug("request is generated for a peer with another public key")
            return False
        with self._nonce_lock:
            current_time = get_dht_time()
            if abs(auth.time - current_time) > self._MAX_CLIENT_SERVICER_TIME_DIFF.total_seconds():
                logger.debug("clocks are not synchronized or a previous request is replayed again")
                return False
            if auth.nonce in self._recent_nonces:
                logger.debug("previous request is replayed again")
                return False
            self._recent_nonces.store(auth.nonce, None, current_time + self._MAX_CLIENT_SERVICER_TIME_DIFF.total_seconds() * 3)
        return True

    async def sign_response(self, response: AuthorizedResponseBase, request: AuthorizedRequestBase) -> None:
        await self.refresh_token_if_needed()
        auth = response.auth
        auth.service_access_token.CopyFrom(self._local_access_token)
        auth.nonce = request.auth.nonce
        assert auth.signature == b""
        auth.signature = self._local_private_key.sign(response.SerializeToString())

    async def validate_response(self, response: AuthorizedResponseBase, request: AuthorizedRequestBase) -> bool:
        await self.refresh_token_if_needed()
        auth = response.auth
        if not self.is_token_valid(auth.service_access_token):
            logger.debug("service failed to prove that it (still) has access to the network")
            return False
        service_public_key = RSAPublicKey.from_bytes(auth.service_access_token.public_key)
        signature = auth.signature
        auth.signature = b""
        if not service_public_key.verify(response.SerializeToString(), signature):
            logger.debug("response has invalid signature")
            return False
        if auth.nonce != request.auth.nonce:
            logger.debug("response is generated for another request")
            return False
        return True


class AuthRole(Enum):
    CLIENT = 0
    SERVICER = 1


class AuthRPCWrapper:
    """Wraps a stub (CLIENT) or a servicer (SERVICER) so that every ``rpc_*`` call is signed and verified."""

    def __init__(self, stub, role: AuthRole, authorizer: Optional[AuthorizerBase],
                 service_public_key: Optional[RSAPublicKey] = None):
        self._stub = stub
        self._role = role
        self._authorizer = authorizer
        self._service_public_key = service_public_key

    def __getattribute__(self, name: str):
        if not name.startswith("rpc_"):
            return object.__getattribute__(self, name)
        stub = object.__getattribute__(self, "_stub")
        method = getattr(stub, name)
        role = object.__getattribute__(self, "_role")
        authorizer = object.__getattribute__(self, "_authorizer")
        service_public_key = object.__getattribute__(self, "_service_public_key")
        if authorizer is None:
            return method

        if inspect.isasyncgenfunction(method):
            @functools.wraps(method)
            async def wrapped_stream(request, *args, **kwargs):
                if role == AuthRole.SERVICER and not await authorizer.validate_request(request):
                    return
                async for item in method(request, *args, **kwargs):
                    if role == AuthRole.SERVICER:
                        await authorizer.sign_response(item, request)
                    yield item

            return wrapped_stream

        @functools.wraps(method)
        async def wrapped_rpc(request: AuthorizedRequestBase, *args, **kwargs):
            if role == AuthRole.CLIENT:
                await authorizer.sign_request(request, service_public_key)
            elif role == AuthRole.SERVICER:
                if not await authorizer.validate_request(request):
                    return None
            response = await method(request, *args, **kwargs)
            if role == AuthRole.SERVICER:
                await authorizer.sign_response(response, request)
            elif role == AuthRole.CLIENT:
                if not await authorizer.validate_response(response, request):
                    return None
            return response

        return wrapped_rpc
