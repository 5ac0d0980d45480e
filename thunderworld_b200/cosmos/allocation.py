"""Budget-constrained choice of one measured repair combination per operator.

Mirrors packages/fp4-repair/src/thunderworld_fp4/cosmos/allocation.py:10-56 (nondominated, allocate): every
operator ("group") offers candidate combinations with an issued-MMA cost and a measured loss; one is chosen per
group so that the total cost stays within budget x base cost. Greedy growth by loss reduction per extra MMA, or
pruning from the best combination down to the cap, followed by bounded rounds of re-growth. Candidate dicts carry
`id`, `base_mma`, `mma`, `loss` and optionally `a_blocks`, `w_blocks`, `qk_counts`, `pv_counts`.
"""
from fractions import Fraction


def nondominated(choices):
    """Candidates that no other candidate beats or ties on both cost and loss while beating one."""
    def beaten(c):
        return any(d['mma'] <= c['mma'] and d['loss'] <= c['loss'] and (d['mma'] < c['mma'] or d['loss'] < c['loss'])
                   for d in choices)
    return [c for c in choices if not beaten(c)]


def _eligible(candidate, preference):
    attention = any(candidate.get('qk_counts', ())) or any(candidate.get('pv_counts', ()))
    if preference == 'a':
        return not candidate.get('w_blocks') and not attention
    if preference == 'w':
        return not candidate.get('a_blocks', 0) and not attention
    return True


def allocate(groups, budget, *, direction='grow', preference=None, rounds=3):
    if direction not in ('grow', 'prune') or not 1 <= rounds <= 3:
        raise ValueError('Invalid search controls')
    # the restriction is applied before the Pareto filter: a dominated candidate may be the best eligible one
    groups = {k: nondominated([c for c in v if _eligible(c, preference)]) for k, v in groups.items()}
    if any(not v for v in groups.values()):
        raise ValueError('Empty candidate group')
    base = sum(min(c['base_mma'] for c in v) for v in groups.values())
    cap = Fraction(str(budget)) * base
    start = (lambda c: (c['mma'], c['loss'])) if direction == 'grow' else (lambda c: (c['loss'], c['mma']))
    chosen = {k: min(v, key=start) for k, v in groups.items()}
    total = lambda: sum(c['mma'] for c in chosen.values())
    if direction == 'prune':
        while total() > cap:
            moves = [((c['loss'] - old['loss']) / (old['mma'] - c['mma']), k, c)
                     for k, old in chosen.items() for c in groups[k] if old['mma'] > c['mma']]
            if not moves:
                raise ValueError('Mandatory supports exceed budget')
            _, key, new = min(moves, key=lambda x: (x[0], x[1], x[2]['id']))
            chosen[key] = new
    for _ in range(rounds):
        changed = False
        while True:
            cost = total()
            moves = []
            for k, old in chosen.items():
                for c in groups[k]:
                    extra, gain = c['mma'] - old['mma'], old['loss'] - c['loss']
                    if gain > 0 and cost + extra <= cap:
                        moves.append((gain / max(extra, 1), gain, k, c))
            if not moves:
                break
            _, _, key, new = max(moves, key=lambda x: (x[0], x[1], x[2], -x[3]['id']))
            chosen[key] = new
            changed = True
        if not changed:
            break
    if total() > cap:
        raise ValueError('Allocator violated budget')
    return dict(base_mma=base, total_mma=total(), ratio=total() / base, budget=budget,
                proxy_loss=sum(c['loss'] for c in chosen.values()), assignments=chosen, direction=direction,
                preference=preference, objective_scope='Measured operator combinations; full trajectory gate required')
