"""Protocol table of the multiaddr subset (codes from the multiformats registry)."""
P_IP4 = 0x04
P_TCP = 0x06
P_DNS = 0x35
P_DNS4 = 0x36
P_DNS6 = 0x37
P_DNSADDR = 0x38
P_IP6 = 0x29
P_UDP = 0x0111
P_P2P_CIRCUIT = 0x0122
P_UNIX = 0x0190
P_P2P = 0x01A5
P_HTTPS = 0x01BB
P_TLS = 0x01C0
P_QUIC = 0x01CC
P_QUIC_V1 = 0x01CD
P_WS = 0x01DD
P_WSS = 0x01DE
P_HTTP = 0x01E0

# size: bits of a fixed-size value, 0 = no value, -1 = length-prefixed value
TABLE = [
    (P_IP4, "ip4", 32), (P_TCP, "tcp", 16), (P_UDP, "udp", 16), (P_IP6, "ip6", 128), (P_DNS, "dns", -1),
    (P_DNS4, "dns4", -1), (P_DNS6, "dns6", -1), (P_DNSADDR, "dnsaddr", -1), (P_UNIX, "unix", -1), (P_P2P, "p2p", -1),
    (P_P2P_CIRCUIT, "p2p-circuit", 0), (P_QUIC, "quic", 0), (P_QUIC_V1, "quic-v1", 0), (P_WS, "ws", 0),
    (P_WSS, "wss", 0), (P_TLS, "tls", 0), (P_HTTP, "http", 0), (P_HTTPS, "https", 0),
]
