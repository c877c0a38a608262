"""Token authorization: valid exchanges, expired tokens, forged signatures, replays, wrong recipient, and the RPC
wrapper in both roles (modelled on the reference's tests/test_auth.py)."""
import asyncio
from datetime import datetime, timedelta, timezone
from typing import Optional


from hivemind_b200.proto import dht_pb2
from hivemind_b200.proto.auth_pb2 import AccessToken
from hivemind_b200.utils.auth import AuthRole, AuthRPCWrapper, TokenAuthorizerBase
from hivemind_b200.utils.crypto import RSAPrivateKey


class MockAuthorizer(TokenAuthorizerBase):
    _authority_private_key = None
    _authority_public_key = None

    def __init__(self, local_private_key: Optional[RSAPrivateKey], username: str = "mock"):
        super().__init__(local_private_key)
        self._username = username
        self._authority_public_key = None

    async def get_token(self) -> AccessToken:
        if MockAuthorizer._authority_private_key is None:
            MockAuthorizer._authority_private_key = RSAPrivateKey()
        self._authority_public_key = MockAuthorizer._authority_private_key.get_public_key()
        token = AccessToken(username=self._username, public_key=self.local_public_key.to_bytes(),
                            expiration_time=str(datetime.now(timezone.utc) + timedelta(minutes=1)))
        token.signature = MockAuthorizer._authority_private_key.sign(self._token_to_bytes(token))
        return token

    def is_token_valid(self, access_token: AccessToken) -> bool:
        data = self._token_to_bytes(access_token)
        if not self._authority_public_key.verify(data, access_token.signature):
            return False
        return datetime.fromisoformat(access_token.expiration_time) >= datetime.now(timezone.utc)

    _MAX_LATENCY = timedelta(minutes=1)

    def does_token_need_refreshing(self, access_token: AccessToken) -> bool:
        return datetime.fromisoformat(access_token.expiration_time) < datetime.now(timezone.utc) + self._MAX_LATENCY

    @staticmethod
    def _token_to_bytes(access_token: AccessToken) -> bytes:
        return f"{access_token.username} {access_token.public_key} {access_token.expiration_time}".encode()


def run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


def test_valid_request_and_response():
    async def scenario():
        client, service = MockAuthorizer(RSAPrivateKey()), MockAuthorizer(RSAPrivateKey())
        request = dht_pb2.PingRequest()
        request.peer.node_id = b"ping"
        await client.sign_request(request, service.local_public_key)
        assert await service.validate_request(request)
        response = dht_pb2.PingResponse()
        response.peer.node_id = b"pong"
        await service.sign_response(response, request)
        assert await client.validate_response(response, request)
    run(scenario())


def test_invalid_access_token():
    async def scenario():
        client, service = MockAuthorizer(RSAPrivateKey()), MockAuthorizer(RSAPrivateKey())
        request = dht_pb2.PingRequest()
        request.peer.node_id = b"ping"
        await client.sign_request(request, service.local_public_key)
        request.auth.client_access_token.username = "another"  # the authority never signed this
        assert not await service.validate_request(request)
        response = dht_pb2.PingResponse()
        await service.sign_response(response, request)
        response.auth.service_access_token.public_key = RSAPrivateKey().get_public_key().to_bytes()
        assert not await client.validate_response(response, request)
    run(scenario())


def test_invalid_signatures_and_recipient():
    async def scenario():
        client, service, other = (MockAuthorizer(RSAPrivateKey()) for _ in range(3))
        request = dht_pb2.PingRequest()
        request.peer.node_id = b"true"
        await client.sign_request(request, service.local_public_key)
        request.peer.node_id = b"fake"  # tampered after signing
        assert not await service.validate_request(request)

        request = dht_pb2.PingRequest()
        await client.sign_request(request, service.local_public_key)
        await other.refresh_token_if_needed()
        assert not await other.validate_request(request)  # meant for another service key

        request = dht_pb2.PingRequest()
        await client.sign_request(request, service.local_public_key)
        response = dht_pb2.PingResponse()
        response.peer.node_id = b"true"
        await service.sign_response(response, request)
        response.peer.node_id = b"fake"
        assert not await client.validate_response(response, request)
    run(scenario())


def test_replay_and_mismatched_nonce():
    async def scenario():
        client, service = MockAuthorizer(RSAPrivateKey()), MockAuthorizer(RSAPrivateKey())
        request = dht_pb2.PingRequest()
        await client.sign_request(request, service.local_public_key)
        replayed = dht_pb2.PingRequest()
        replayed.CopyFrom(request)
        assert await service.validate_request(request)
        assert not await service.validate_request(replayed)  # same nonce again

        first, second = dht_pb2.PingRequest(), dht_pb2.PingRequest()
        await client.sign_request(first, service.local_public_key)
        await client.sign_request(second, service.local_public_key)
        response = dht_pb2.PingResponse()
        await service.sign_response(response, first)
        assert not await client.validate_response(response, second)  # answers a different request

        late = dht_pb2.PingRequest()
        await client.sign_request(late, service.local_public_key)
        late.auth.signature = b""
        late.auth.time -= 3600  # an hour-old request, re-signed by the client itself
        late.auth.signature = client._local_private_key.sign(late.SerializeToString())
        assert not await service.validate_request(late)
    run(scenario())


def test_rpc_wrapper_roles():
    class Servicer:
        async def rpc_increment(self, request: dht_pb2.PingRequest) -> dht_pb2.PingResponse:
            assert request.peer.node_id == b"ping" and request.auth.client_access_token.username == "alice"
            response = dht_pb2.PingResponse()
            response.peer.node_id = b"pong"
            return response

    class Client:
        def __init__(self, servicer):
            self._servicer = servicer

        async def rpc_increment(self, request: dht_pb2.PingRequest) -> dht_pb2.PingResponse:
            return await self._servicer.rpc_increment(request)

    async def scenario():
        service_auth = MockAuthorizer(RSAPrivateKey(), "bob")
        servicer = AuthRPCWrapper(Servicer(), AuthRole.SERVICER, service_auth)
        client = AuthRPCWrapper(Client(servicer), AuthRole.CLIENT, MockAuthorizer(RSAPrivateKey(), "alice"),
                                service_public_key=service_auth.local_public_key)
        request = dht_pb2.PingRequest()
        request.peer.node_id = b"ping"
        response = await client.rpc_increment(request)
        assert response.peer.node_id == b"pong" and response.auth.service_access_token.username == "bob"

        stranger = AuthRPCWrapper(Client(servicer), AuthRole.CLIENT, MockAuthorizer(RSAPrivateKey(), "alice"),
                                  service_public_key=RSAPrivateKey().get_public_key())
        request = dht_pb2.PingRequest()
        request.peer.node_id = b"ping"
        assert await stranger.rpc_increment(request) is None  # addressed to the wrong service: no answer

        passthrough = AuthRPCWrapper(Servicer(), AuthRole.SERVICER, None)
        assert passthrough.rpc_increment.__self__.__class__ is Servicer
    run(scenario())
