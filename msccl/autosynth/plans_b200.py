"""Plans for a single HGX B200 box (machine type ``b200``): 2, 4 or 8 GPUs behind NVSwitch.

Size ranges follow the latency/bandwidth trade-off of the algorithms: one-shot while latency
dominates, two-shot in the middle, and for large messages the in-switch (NVLS) reduction,
which the executor provides natively (``msccl.language.ext_nvls``).
"""
from msccl.autosynth.registry import register_msccl_program, register_synthesis_plan
from msccl.language.mscclir import ThreadblockPolicy
from msccl.programs.allgather import allgather_direct, reduce_scatter_direct
from msccl.programs.allreduce import allreduce_one_shot, allreduce_ring, allreduce_two_shot
from msccl.programs.alltoall import alltoall_direct
from msccl.language.ext_nvls import allreduce_nvls
from msccl.topologies import fully_connected

B200_GPU_COUNTS = (2, 4, 8)


def register_b200_plans():
    manual = ThreadblockPolicy.manual
    # One CTA moves roughly 50 GB/s, so a plan needs a few dozen CTAs per direction to fill a GPU's
    # NVLink port; all threadblocks of a plan must also be co-resident (148 SMs).
    # Measured on two GPUs (a send and a receive threadblock per copy and peer): all-gather of 64 MB 114 us with 32
    # copies, 87 us with 64 (NCCL 100 us); all-to-all of 64 MB 121 -> 88 us (NCCL 126 us).
    copies = {2: 64, 4: 16, 8: 8}
    # The two-shot all-reduce has one threadblock per copy and peer and reduces locally between its two transfers:
    # 256 MB on two GPUs took 634 / 510 / 482 us with 32 / 64 / 128 copies (NCCL 526 us), on four GPUs 1132 / 918 us with
    # 16 / 32 copies (NCCL 682 us, which reduces inside the switch; so does the in-switch program of
    # msccl.language.ext_nvls on registered tensors: 604 us); on eight GPUs 64 MB took 617 / 396 us with 8 / 16 copies.
    reduce_copies = {2: 128, 4: 32, 8: 16}
    small = {2: 4, 4: 2, 8: 1}     # latency-bound sizes: flag-in-data packets, few CTAs
    # between the two: 128-byte lines with 120 bytes of payload (LL128), no fence per tile; ahead of the Simple plans up
    # to 1-2 MB on two GPUs (all-gather of 1 MB: 20.5 us against 22.1 us), behind them from 4 MB
    middle = {2: 16, 4: 8, 8: 4}
    for n in B200_GPU_COUNTS:
        mtype = f'b200x{n}' if n != 8 else ['b200', 'b200x8']
        box = fully_connected(n)

        def one_shot(prog, nodes, n=n):
            allreduce_one_shot(n)
        one_shot.__name__ = f'b200_allreduce_one_shot_{n}'
        register_msccl_program(box, 'allreduce', mtype, chunk_factor=1, inplace=True, protocol='LL',
                               sizes=(0, '256KB' if n > 2 else '32KB'), threadblock_policy=manual,
                               machines=lambda m: m == 1)(one_shot)

        def two_shot(prog, nodes, n=n):
            allreduce_two_shot(n)
        two_shot.__name__ = f'b200_allreduce_two_shot_{n}'

        def two_shot_ll128(prog, nodes, n=n):
            allreduce_two_shot(n)
        two_shot_ll128.__name__ = f'b200_allreduce_two_shot_ll128_{n}'
        if n > 2:
            register_msccl_program(box, 'allreduce', mtype, chunk_factor=n, inplace=True, protocol='Simple',
                                   sizes=('256KB', None), instances=reduce_copies[n], threadblock_policy=manual,
                                   machines=lambda m: m == 1)(two_shot)
            register_msccl_program(box, 'allreduce', mtype, chunk_factor=n, inplace=True, protocol='LL128',
                                   sizes=('256KB', '1MB'), instances=middle[n], threadblock_policy=manual,
                                   machines=lambda m: m == 1)(two_shot_ll128)
            # From 4 GPUs up the reduction belongs into the switch: the program of in-switch steps (one multimem
            # load-reduce and one multimem store per vector; `msccl.language.ext_nvls`) is what NCCL's NVLS algorithm
            # does too, and no program of peer stores can match it.  Against NCCL on registered tensors: x1.1-1.8 from
            # 64 KB to 256 MB on 8 GPUs, x0.8-0.9 below 1 MB and x1.1-2.3 above on 4 GPUs, where the two-shot program over
            # peer stores reaches x0.4-0.75.  Tensors that are not registered memory pass through registered staging
            # slices (8 GPUs: x1.4 at 16 MB, x0.98 at 256 MB).  The peer-store programs stay registered underneath for
            # the sizes below.
            def in_switch(machines, n=n):
                return allreduce_nvls(n, 8, name=f'b200_allreduce_in_switch_{n}')
            in_switch.__name__ = f'b200_allreduce_in_switch_{n}'
            register_synthesis_plan('allreduce', mtype, machines=lambda m: m == 1, sizes=('64KB', None))(in_switch)
        else:
            # Two GPUs: the ring on two channels is the two-shot exchange with the receive, the reduction and the
            # send back fused into one step (three steps per threadblock instead of five).  Measured against NCCL
            # on the same box:
            #   LL, 128 threadblocks      20.0 / 18.9 / 20.3 us at 64 KB / 256 KB / 1 MB   (NCCL 20.8 / 20.4 / 20.8)
            #   LL128, 128 threadblocks   27.7 us at 4 MB                                   (NCCL 40.7; Simple 33.8; LL 33.4)
            #   Simple, 128 threadblocks  61 / 157 / 492 us at 16 / 64 / 256 MB             (NCCL 62 / 167 / 549)
            for proto, low, high, inst in (('LL', '32KB', '2MB', 64), ('LL128', '2MB', '8MB', 64),
                                           ('Simple', '8MB', None, reduce_copies[2] // 2)):
                def ring(prog, nodes):
                    allreduce_ring(2, 2)
                ring.__name__ = 'b200_allreduce_ring_2' + {'LL': '_ll', 'LL128': '_ll128', 'Simple': ''}[proto]
                register_msccl_program(box, 'allreduce', mtype, chunk_factor=2, inplace=True, protocol=proto,
                                       sizes=(low, high), instances=inst, threadblock_policy=manual,
                                       machines=lambda m: m == 1)(ring)

        def a2a(prog, nodes, n=n):
            alltoall_direct(n)
        a2a.__name__ = f'b200_alltoall_direct_{n}'
        register_msccl_program(box, 'alltoall', mtype, chunk_factor=1, protocol='Simple', instances=copies[n],
                               sizes=('512KB', None), machines=lambda m: m == 1)(a2a)


        def a2a_ll(prog, nodes, n=n):
            alltoall_direct(n)
        a2a_ll.__name__ = f'b200_alltoall_direct_ll_{n}'
        register_msccl_program(box, 'alltoall', mtype, chunk_factor=1, protocol='LL', instances=small[n],
                               sizes=(0, '512KB'), machines=lambda m: m == 1)(a2a_ll)

        def ag(prog, nodes, n=n):
            allgather_direct(n)
        ag.__name__ = f'b200_allgather_direct_{n}'
        register_msccl_program(box, 'allgather', mtype, chunk_factor=1, protocol='Simple', instances=copies[n],
                               sizes=('512KB', None), machines=lambda m: m == 1)(ag)

        def ag_ll(prog, nodes, n=n):
            allgather_direct(n)
        ag_ll.__name__ = f'b200_allgather_direct_ll_{n}'
        register_msccl_program(box, 'allgather', mtype, chunk_factor=1, protocol='LL', instances=small[n],
                               sizes=(0, '512KB'), machines=lambda m: m == 1)(ag_ll)

        def rs(prog, nodes, n=n):
            reduce_scatter_direct(n)
        rs.__name__ = f'b200_reduce_scatter_direct_{n}'
        register_msccl_program(box, 'reduce_scatter', mtype, chunk_factor=1, protocol='Simple', instances=copies[n],
                               sizes=('512KB', None), machines=lambda m: m == 1)(rs)

        def rs_ll(prog, nodes, n=n):
            reduce_scatter_direct(n)
        rs_ll.__name__ = f'b200_reduce_scatter_direct_ll_{n}'
        register_msccl_program(box, 'reduce_scatter', mtype, chunk_factor=1, protocol='LL', instances=small[n],
                               sizes=(0, '512KB'), machines=lambda m: m == 1)(rs_ll)

        # registered last: on equal ranges the later registration wins
        def a2a_ll128(prog, nodes, n=n):
            alltoall_direct(n)
        a2a_ll128.__name__ = f'b200_alltoall_direct_ll128_{n}'
        register_msccl_program(box, 'alltoall', mtype, chunk_factor=1, protocol='LL128', instances=middle[n],
                               sizes=('512KB', '2MB'), machines=lambda m: m == 1)(a2a_ll128)

        def ag_ll128(prog, nodes, n=n):
            allgather_direct(n)
        ag_ll128.__name__ = f'b200_allgather_direct_ll128_{n}'
        register_msccl_program(box, 'allgather', mtype, chunk_factor=1, protocol='LL128', instances=middle[n],
                               sizes=('512KB', '2MB'), machines=lambda m: m == 1)(ag_ll128)

        def rs_ll128(prog, nodes, n=n):
            reduce_scatter_direct(n)
        rs_ll128.__name__ = f'b200_reduce_scatter_direct_ll128_{n}'
        register_msccl_program(box, 'reduce_scatter', mtype, chunk_factor=1, protocol='LL128', instances=middle[n],
                               sizes=('512KB', '2MB'), machines=lambda m: m == 1)(rs_ll128)
