"""CPU model of the barrier protocol of the W4A16 tensor-memory kernel
(kernel_set_b200/csrc/sm100_w4a16.cu, TA path): every role of one CTA (weight and
activation producers, MMA issuers, dequantisation groups, epilogue) as a coroutine, every
mbarrier with its arrival count and the exact phase parities the kernel waits on. Running
all roles to completion for every CTA of a launch shows that the protocol cannot deadlock
and that no wait can alias a phase; it is a check of the protocol's logic, not of timing.
The model must be kept in step with the kernel by hand.

What it caught: with THREE issuers and four operand stages the issuer of unit it + 4 is not
the issuer of unit it, so nothing orders its wait on deq_full[stage] (parity of the second
use) after the first use has completed; on a fresh barrier that wait passes at once and the
issuer multiplies an operand stage that is still being written. On the GPU this showed as
an intermittent bounded-wait timeout on the first large launch of a process. The number of
operand and activation stages must be a multiple of the number of issuers."""
import pytest

class Bar:
    def __init__(s, count): s.count=count; s.pending=count; s.phase=0
    def arrive(s):
        s.pending-=1
        assert s.pending>=0
        if s.pending==0: s.phase+=1; s.pending=s.count
    def done(s, parity): return (s.phase & 1) != parity
def run_start(units, ctas, c): return (units*c)//ctas
def sim_cta(ub, ue, k_steps, K=2, G=4, RS=8, AS=8, DS=4, order=None):
    raw_full=[Bar(1) for _ in range(RS)]; raw_empty=[Bar(2) for _ in range(RS)]
    act_full=[Bar(1) for _ in range(AS)]; act_empty=[Bar(1) for _ in range(AS)]
    deq_full=[Bar(1) for _ in range(DS)]; deq_empty=[Bar(1) for _ in range(DS)]
    acc_full=[Bar(K) for _ in range(2)]; acc_empty=[Bar(1) for _ in range(2)]
    b_begin, b_end = ub>>1, (ue+1)>>1
    def wprod():
        itb=0
        for b in range(b_begin,b_end):
            sr=itb%RS; pr=(itb//RS)&1
            yield ('wait', raw_empty[sr], pr^1, itb//RS, 'wprod raw_empty')
            raw_full[sr].arrive()
            itb+=1
    def aprod():
        it=0
        for u in range(ub,ue):
            sa=it%AS; pa=(it//AS)&1
            yield ('wait', act_empty[sa], pa^1, it//AS, 'aprod act_empty')
            act_full[sa].arrive()
            it+=1
    def issuer(i):
        it=0; seg=0; n_in_seg=0; step=ub%k_steps
        for u in range(ub,ue):
            seg_first=(u==ub) or step==0
            seg_last=(u+1==ue) or step==k_steps-1
            tile_last=u-step+k_steps-1
            seg_last_u=min(tile_last,ue-1)
            mine=(it%K)==i
            my_last=u+K>seg_last_u
            sd=it%DS; pd=(it//DS)&1; sa=it%AS; pa=(it//AS)&1
            buf=seg&1; pacc=(seg>>1)&1
            if seg_first: n_in_seg=0
            if mine:
                if n_in_seg==0: yield ('wait', acc_empty[buf], pacc^1, seg>>1, f'issuer{i} acc_empty u={u}')
                yield ('wait', deq_full[sd], pd, it//DS+1, f'issuer{i} deq_full u={u}')
                yield ('wait', act_full[sa], pa, it//AS+1, f'issuer{i} act_full u={u}')
                n_in_seg+=1
                deq_empty[sd].arrive(); act_empty[sa].arrive()
                if my_last: acc_full[buf].arrive()
            elif seg_last and n_in_seg==0:
                yield ('wait', acc_empty[buf], pacc^1, seg>>1, f'issuer{i} idle acc_empty u={u}')
                acc_full[buf].arrive()
            if seg_last: seg+=1
            it+=1; step=0 if step+1==k_steps else step+1
    def group(g):
        stride=G//2; half=g&1
        b=b_begin
        while (b%stride)!=(g>>1): b+=1
        while b<b_end:
            itb=b-b_begin; sr=itb%RS; pr=(itb//RS)&1
            u=2*b+half
            if u<ub or u>=ue:
                raw_empty[sr].arrive(); b+=stride; continue
            it=u-ub; sd=it%DS; pd=(it//DS)&1
            yield ('wait', raw_full[sr], pr, itb//RS+1, f'group{g} raw_full u={u}')
            yield ('wait', deq_empty[sd], pd^1, it//DS, f'group{g} deq_empty u={u}')
            raw_empty[sr].arrive()
            deq_full[sd].arrive()
            b+=stride
    def epilogue():
        seg=0; u=ub
        while u<ue:
            step0=u%k_steps
            tile_end=u-step0+k_steps
            seg_end=min(tile_end,ue)
            buf=seg&1; pacc=(seg>>1)&1
            seg+=1; u=seg_end
            yield ('wait', acc_full[buf], pacc, ((seg-1)>>1)+1, f'epilogue acc_full seg={seg-1}')
            acc_empty[buf].arrive()
    procs={'wprod':wprod(),'aprod':aprod(),'epi':epilogue()}
    for i in range(K): procs[f'iss{i}']=issuer(i)
    for g in range(G): procs[f'grp{g}']=group(g)
    blocked={}
    alive=list(procs)
    if order is not None:
        order.shuffle(alive)
    problems={}
    while alive:
        progressed=False
        for name in list(alive):
            gen=procs[name]
            while True:
                if name in blocked:
                    bar,par,want,desc=blocked[name]
                    if not bar.done(par): break
                    if bar.phase!=want: problems[name]=f'{desc}: passed at completion {bar.phase}, meant {want}'
                    del blocked[name]; progressed=True
                try:
                    op=next(gen)
                except StopIteration:
                    alive.remove(name); progressed=True; break
                _,bar,par,want,desc=op
                if bar.done(par):
                    if bar.phase!=want: problems[name]=f'{desc}: passed at completion {bar.phase}, meant {want}'
                    progressed=True; continue
                blocked[name]=(bar,par,want,desc); break
        if not progressed:
            problems.update({n:'stuck at '+blocked[n][3] for n in blocked})
            return problems
    return problems or None


def deadlocked_ctas(n_tiles, k_steps, ctas=148, **kw):
    """CTAs whose roles get stuck or pass a wait at the wrong phase, under the natural role
    order and under a few shuffled ones (the protocol must not depend on who runs first)."""
    import random
    units = n_tiles * k_steps
    ctas = min(ctas, units)
    stuck = []
    for c in range(ctas):
        ub, ue = run_start(units, ctas, c), run_start(units, ctas, c + 1)
        for order in (None, random.Random(1), random.Random(2), random.Random(3)):
            r = sim_cta(ub, ue, k_steps, order=order, **kw)
            if r:
                stuck.append((c, ub, ue, r))
                break
    return stuck


@pytest.mark.parametrize("n_tiles,k_steps", [
    (224, 32),    # K=4096, N=28672: ~48 units per CTA
    (32, 112),    # K=14336, N=4096
    (112, 32),    # ~24 units per CTA
    (28, 32), (2, 8), (5, 2), (1, 2), (3, 6), (37, 4),
])
@pytest.mark.parametrize("issuers,groups", [(2, 4), (2, 2), (4, 4)])
def test_protocol_runs_to_completion(n_tiles, k_steps, issuers, groups):
    assert deadlocked_ctas(n_tiles, k_steps, K=issuers, G=groups) == []


def test_every_issuer_arrives_once_per_segment():
    """acc_full expects exactly one arrival per issuer and segment (a commit after the
    issuer's last unit of the segment, or a plain arrival when it owns none)."""
    for (n_tiles, k_steps, issuers) in ((224, 32, 2), (224, 32, 4), (5, 2, 2), (5, 2, 4), (32, 112, 2)):
        units = n_tiles * k_steps
        ctas = min(148, units)
        for c in range(ctas):
            ub, ue = run_start(units, ctas, c), run_start(units, ctas, c + 1)
            for issuer in range(issuers):
                it = seg = n_in_seg = 0
                step = ub % k_steps
                arrivals = {}
                for u in range(ub, ue):
                    seg_first = (u == ub) or step == 0
                    seg_last = (u + 1 == ue) or step == k_steps - 1
                    seg_last_u = min(u - step + k_steps - 1, ue - 1)
                    mine = (it % issuers) == issuer
                    if seg_first:
                        n_in_seg = 0
                    if mine:
                        n_in_seg += 1
                        if u + issuers > seg_last_u:
                            arrivals[seg] = arrivals.get(seg, 0) + 1
                    elif seg_last and n_in_seg == 0:
                        arrivals[seg] = arrivals.get(seg, 0) + 1
                    if seg_last:
                        seg += 1
                    it += 1
                    step = 0 if step + 1 == k_steps else step + 1
                assert all(arrivals.get(sg, 0) == 1 for sg in range(seg)), (n_tiles, k_steps, issuers, c, issuer)


def test_three_issuers_are_detected_as_broken():
    """The configuration that failed on the GPU fails in the model too."""
    assert deadlocked_ctas(28, 32, K=3, G=4) != []
