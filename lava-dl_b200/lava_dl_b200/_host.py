"""Host-side placement for pinned staging buffers.

Streaming batches between host memory and a GPU runs at PCIe speed only when
the pinned pages sit on the NUMA node the GPU hangs off: on a two-socket host
with eight GPUs, buffers that land on the other socket cross the inter-socket
link in both directions and eight ranks then share that link.  ``bind_near_gpu``
asks the kernel (a) to prefer the GPU's node for this process's future page
allocations and (b) to run this process on that node's cores, as far as the
container's cpuset allows.  Both are properties of the calling process only;
nothing about the GPU or the machine is changed, and every step is optional
(a missing sysfs entry or a refused call leaves the process as it was).

The reference has no counterpart: it has no host-streaming path at all.
"""

import ctypes
import os

MPOL_PREFERRED = 1
_SYS_SET_MEMPOLICY = 238  # x86_64


def _pci_address(device_index):
    import torch
    p = torch.cuda.get_device_properties(device_index)
    try:
        return f'{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0'
    except AttributeError:
        return None


def _read(path):
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def _parse_cpulist(text):
    cpus = set()
    for part in (text or '').split(','):
        part = part.strip()
        if not part:
            continue
        if '-' in part:
            lo, hi = part.split('-')
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_numa_node(device_index):
    """NUMA node of the GPU (from sysfs, read-only) or ``None`` when unknown."""
    addr = _pci_address(device_index)
    if addr is None:
        return None
    txt = _read(f'/sys/bus/pci/devices/{addr}/numa_node')
    try:
        node = int(txt)
    except (TypeError, ValueError):
        return None
    return node if node >= 0 else None


def bind_near_gpu(device_index):
    """Prefer the GPU's NUMA node for memory and CPU placement of this process.

    Call it before allocating pinned buffers.  Returns a dict that says what was
    found and what took effect: ``node``, ``mempolicy`` (True when the kernel
    accepted the preference), ``cpus`` (the affinity set now in force, or
    ``None`` when it was left alone)."""
    info = {'node': gpu_numa_node(device_index), 'mempolicy': False, 'cpus': None, 'previous_cpus': None}
    node = info['node']
    if node is None:
        return info
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        nbits = 64 * (node // 64 + 1)
        mask = (ctypes.c_ulong * (nbits // 64))()
        mask[node // 64] = 1 << (node % 64)
        rc = libc.syscall(_SYS_SET_MEMPOLICY, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(nbits + 1))
        info['mempolicy'] = rc == 0
    except (OSError, AttributeError):
        pass
    try:
        allowed = os.sched_getaffinity(0)
        local = _parse_cpulist(_read(f'/sys/devices/system/node/node{node}/cpulist')) & allowed
        if local and local != allowed:
            os.sched_setaffinity(0, local)
            info['cpus'] = sorted(local)
            info['previous_cpus'] = sorted(allowed)
    except (OSError, AttributeError):
        pass
    return info


def restore_affinity(info):
    """Undo the CPU part of ``bind_near_gpu`` (the memory preference only matters for new pages)."""
    if info.get('previous_cpus'):
        try:
            os.sched_setaffinity(0, set(info['previous_cpus']))
        except OSError:
            pass
