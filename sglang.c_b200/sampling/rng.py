"""The reference's generator: xorshift64* (src/sampling.c:10-21) with the
request's stream seeded through mix64 (src/scheduler.c:95-100,195).  The
reference ignores the caller's seed; here it is mixed in."""
_M = (1 << 64) - 1


def mix64(x):
    x &= _M
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & _M
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & _M
    x ^= x >> 33
    return x


def request_stream(seed, request_id):
    """Initial state of a request's generator; never zero."""
    s = mix64((int(seed) & _M) ^ mix64((int(request_id) * 0x9E3779B97F4A7C15 + 1) & _M))
    return s or 0x9E3779B97F4A7C15


def next_u64(state):
    x = state & _M
    x ^= x >> 12
    x ^= (x << 25) & _M
    x ^= x >> 27
    return x, (x * 0x2545F4914F6CDD1D) & _M


def uniform(state):
    """(new state, u) with u = (next >> 11) / 2^53 in [0,1)."""
    state, out = next_u64(state)
    return state, (out >> 11) / 9007199254740992.0
