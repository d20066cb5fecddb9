"""The oracle's softmax and batchnorm against the reference's own known-answer vectors
(test/softmax/softmax_{forward,grad}.cc, test/batchnorm/batchnorm_{forward,gradient}_{frozen,training}.cc:
324 cases, all committed in tests/golden/norm_kat.npz) with the reference fixtures' tolerances."""
import norm_cases


def test_oracle_matches_every_softmax_and_batchnorm_vector(orc):
    cases = norm_cases.load_cases()
    assert len(cases) == 324
    failures = []
    for case in cases:
        for what, ok, err in norm_cases.run_case(case, orc):
            if not ok:
                failures.append((case["op"], case["name"], what, err))
    assert not failures, failures[:10]
