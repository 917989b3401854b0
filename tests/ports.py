"""Rendezvous ports for the multi-process tests.

A port found by binding to 0 comes from the kernel's ephemeral range, from which NCCL, gloo and the
store's own clients draw their outgoing connections all the time: between closing the probe
socket and the ranks' TCPStore listening on it, the port can be taken.  Ports are therefore drawn
below that range, and a launch whose ranks report the address in use is repeated on another port.
"""
import random
import socket

_RANGE = (20000, 32000)        # below Linux's default ephemeral range (32768-60999)


def free_port() -> int:
    rng = random.SystemRandom()
    for _ in range(200):
        port = rng.randrange(*_RANGE)
        with socket.socket() as s:
            try:
                s.bind(("127.0.0.1", port))
            except OSError:
                continue
            return port
    raise RuntimeError("no free rendezvous port found")


def address_in_use(outputs) -> bool:
    """True when a rank's output shows that the rendezvous port was taken."""
    return any(o and ("EADDRINUSE" in o or "address already in use" in o.lower()) for o in outputs)
