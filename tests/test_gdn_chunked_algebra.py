"""CPU check of the algebra behind the chunked (64-token WY form) gated-delta-net recurrence: the closed form the two
kernels of gdn_chunked.cu evaluate -- (I + A) [W | U] = [beta G K | beta V], D = U - W M0, O = diag(G) Q M0 + P D,
M64 = G64 M0 + (diag(G64 / G) K)^T D -- restated in float64 with numpy and compared with the token recurrence
(gated_delta_net_update_reference_cpu, src/runtime/reference/gdn_decode.cpp:186-293, here without any rounding).  In
exact arithmetic the two are the same function; in float64 they agree to 1e-11.  Ragged tails are handled the way the
kernels handle them: a row past the span has beta = 0 and no decay."""
import numpy as np
import pytest

CHUNK = 64


def token_recurrence(q, k, v, alpha, beta, state):
    """q, k [T, dk] (normalised), v [T, dv], alpha / beta [T], state [dk, dv] -> outputs [T, dv], final state."""
    M = state.copy()
    out = np.empty((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        M *= alpha[t]
        delta = beta[t] * (v[t] - M.T @ k[t])
        M += np.outer(k[t], delta)
        out[t] = M.T @ q[t]
    return out, M


def chunked_recurrence(q, k, v, alpha, beta, state):
    T, dk = q.shape
    dv = v.shape[1]
    M = state.copy()
    out = np.empty((T, dv))
    for start in range(0, T, CHUNK):
        live = min(CHUNK, T - start)
        Q, K, V = np.zeros((CHUNK, dk)), np.zeros((CHUNK, dk)), np.zeros((CHUNK, dv))
        Q[:live], K[:live], V[:live] = q[start:start + live], k[start:start + live], v[start:start + live]
        g, b = np.zeros(CHUNK), np.zeros(CHUNK)                      # log-decays and betas; zero past the span
        g[:live], b[:live] = np.log(alpha[start:start + live]), beta[start:start + live]
        c = np.cumsum(g)                                             # log G_t
        ratio = np.exp(c[:, None] - c[None, :])                      # G_t / G_j
        A = np.tril(b[:, None] * ratio * (K @ K.T), -1)
        solve = np.linalg.solve(np.eye(CHUNK) + A, np.concatenate([(b * np.exp(c))[:, None] * K, b[:, None] * V], axis=1))
        W, U = solve[:, :dk], solve[:, dk:]
        D = U - W @ M
        P = np.tril(ratio * (Q @ K.T), 0)
        O = np.exp(c)[:, None] * (Q @ M) + P @ D
        out[start:start + live] = O[:live]
        M = np.exp(c[-1]) * M + (np.exp(c[-1] - c)[:, None] * K).T @ D
    return out, M


@pytest.mark.parametrize("tokens,slow", [(1, False), (63, True), (64, False), (65, True), (200, False), (333, True)])
def test_the_chunked_closed_form_is_the_token_recurrence(tokens, slow):
    rng = np.random.default_rng([tokens, int(slow), 181])
    dk = dv = 32  # the algebra does not depend on the head dimension
    q, k = rng.standard_normal((tokens, dk)), rng.standard_normal((tokens, dk))
    q /= np.linalg.norm(q, axis=1, keepdims=True) * np.sqrt(dk)
    k /= np.linalg.norm(k, axis=1, keepdims=True)
    v = rng.standard_normal((tokens, dv))
    decay = rng.uniform(0.001, 0.05, tokens) if slow else rng.uniform(0.05, 6.0, tokens)
    alpha, beta = np.exp(-decay), 1.0 / (1.0 + np.exp(-2.0 * rng.standard_normal(tokens)))
    state = 0.05 * rng.standard_normal((dk, dv))
    want_out, want_state = token_recurrence(q, k, v, alpha, beta, state)
    got_out, got_state = chunked_recurrence(q, k, v, alpha, beta, state)
    scale_out, scale_state = max(np.abs(want_out).max(), 1e-30), max(np.abs(want_state).max(), 1e-30)
    assert np.abs(got_out - want_out).max() <= 1e-11 * scale_out
    assert np.abs(got_state - want_state).max() <= 1e-11 * scale_state
