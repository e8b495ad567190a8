#include "planner.hpp"

#include <algorithm>
#include <array>

namespace aixb200
{

const char* opName(Op op)
{
    static const char* names[] = {"add", "sub", "mul", "div", "neg", "sqrt", "sin", "cos", "tanh", "log", "exp", "pow",
                                  "fill", "cast", "sumall", "maxall", "sumrows", "maxrows"};
    return names[static_cast<size_t>(op)];
}

Access classifyAccess(const View& v, uint64_t count)
{
    if (v.isBroadcastScalar()) return Access::Scalar;
    if (v.isDense() && v.size == count) return Access::Dense;
    if (v.rank == 2 && v.strides[0] == 0 && v.strides[1] == 1) return Access::RowBcast;
    if (v.rank == 2 && v.strides[1] == 0) return Access::ColBcast;
    return Access::General;
}

namespace
{

struct Group
{
    uint64_t count = 0;
    std::vector<size_t> ops;        // indices into the recorded list, program order
    std::vector<View> loads;        // distinct views this group reads from memory
    size_t liveOutputs = 0;         // results whose storage is still alive (they will be stored)
    size_t reductions = 0;
    uint64_t rowCols = 0;           // row length of the row reductions this group holds (they all share it)
};

// Where an input of a recorded op comes from.
struct InputBinding
{
    enum Kind : uint8_t { Memory, Producer, ImmediateFill } kind = Memory;
    size_t producer = 0;            // op index (Producer / ImmediateFill)
};

bool isOneElementFill(const OpRecord& r) { return r.op == Op::Fill && r.out.size == 1; }

}   // namespace

std::vector<KernelSpec> planKernels(const std::vector<OpRecord>& ops, const std::unordered_set<const void*>& released,
                                    const PlannerLimits& limits)
{
    const size_t n = ops.size();
    std::vector<size_t> groupOf(n, 0);
    std::vector<std::array<InputBinding, 2>> bindings(n);
    std::vector<Group> groups;
    // A fill of a row reduction's destination whose value the reduction takes as a kernel scalar: it is never stored
    // (the reduction writes every element of it) and orders nothing.
    std::vector<char> superseded(n, 0);

    // Byte range every view touches, computed once: the hazard tests below compare ranges, not base pointers (two
    // descriptors may reach one buffer through different bases, e.g. an interior pointer).
    struct Range { const char* lo; const char* hi; };
    auto rangeOf = [](const View& v) { return Range{v.firstByte(), v.endByte()}; };
    auto meet = [](const Range& a, const Range& b) { return a.lo < b.hi && b.lo < a.hi; };
    std::vector<Range> outRange(n);
    std::vector<std::array<Range, 2>> inRange(n);
    for (size_t j = 0; j < n; ++j)
    {
        outRange[j] = rangeOf(ops[j].out);
        for (int k = 0; k < ops[j].numInputs; ++k) inRange[j][k] = rangeOf(ops[j].in[k]);
    }

    // ---- pass 1: dependencies and group placement, in program order -------------------------------------------
    for (size_t j = 0; j < n; ++j)
    {
        const OpRecord& rj = ops[j];
        size_t minGroup = 0;

        for (int k = 0; k < rj.numInputs; ++k)
        {
            const View& in = rj.in[k];
            InputBinding bind;
            bool shadowed = false;      // a more recent writer touches part of the view through a different view
            if (k == 1 && isRowReduction(rj.op))
            {
                // The destination as the reduction's initial value. The usual caller has just filled it (zero, or the
                // lowest value for a maximum): when that fill is still pending, defines every element and nobody has
                // read the destination since, the value travels as a kernel scalar and the fill is dropped. Anything
                // else is read from memory, after the kernels of all pending writers.
                size_t writer = n;
                for (size_t i = j; i-- > 0 && writer == n;)
                    if (meet(outRange[i], inRange[j][1])) writer = i;
                bool immediate = limits.fusion && writer != n && ops[writer].op == Op::Fill && ops[writer].out.sameElements(in);
                for (size_t i = writer + 1; immediate && i < j; ++i)
                    for (int q = 0; q < ops[i].numInputs; ++q)
                        if (meet(inRange[i][q], inRange[j][1])) immediate = false;
                if (immediate)
                {
                    bind.kind = InputBinding::ImmediateFill;
                    bind.producer = writer;
                    superseded[writer] = 1;
                }
                else
                    for (size_t i = 0; i < j; ++i)
                        if (meet(outRange[i], inRange[j][1])) minGroup = std::max(minGroup, groupOf[i] + 1);
                bindings[j][k] = bind;
                continue;
            }
            for (size_t i = j; i-- > 0;)
            {
                const View& w = ops[i].out;
                if (!meet(outRange[i], inRange[j][k])) continue;
                if (isReduction(ops[i].op))
                {
                    // written when the producing grid has finished: readable from the next kernel on
                    shadowed = true;
                    minGroup = std::max(minGroup, groupOf[i] + 1);
                    continue;
                }
                if (!shadowed && isOneElementFill(ops[i]) && in.isBroadcastScalar() && w.dtype == in.dtype &&
                    outRange[i].lo == inRange[j][k].lo)
                {
                    bind.kind = InputBinding::ImmediateFill;     // value known on the host: no ordering needed
                    bind.producer = i;
                    break;
                }
                if (w.sameElements(in))
                {
                    minGroup = std::max(minGroup, groupOf[i]);
                    if (!shadowed) { bind.kind = InputBinding::Producer; bind.producer = i; }
                    break;                                       // this writer defines every element; older ones are hidden
                }
                shadowed = true;
                minGroup = std::max(minGroup, groupOf[i] + 1);   // needs a grid-wide barrier
            }
            bindings[j][k] = bind;
        }

        // write-after-read and write-after-write
        // (a reduction's result is not written element by element: no same-kernel ordering with anything that touches it)
        const bool jReduces = isReduction(rj.op);
        for (size_t i = 0; i < j; ++i)
        {
            const OpRecord& ri = ops[i];
            for (int k = 0; k < ri.numInputs; ++k)
            {
                const View& r = ri.in[k];
                if (!meet(inRange[i][k], outRange[j])) continue;
                minGroup = std::max(minGroup, (r.sameElements(rj.out) && !jReduces) ? groupOf[i] : groupOf[i] + 1);
            }
            if (meet(outRange[i], outRange[j]) && !(superseded[i] && bindings[j][1].kind == InputBinding::ImmediateFill && bindings[j][1].producer == i))
                minGroup = std::max(minGroup, (ri.out.sameElements(rj.out) && !jReduces && !isReduction(ri.op)) ? groupOf[i] : groupOf[i] + 1);
        }

        const uint64_t count = jReduces ? rj.in[0].size : rj.out.size;
        const bool liveOutput = !jReduces && released.count(rj.out.base) == 0;
        // Views op j would have to load if it joined group g: inputs not produced inside g and not loaded by g yet.
        auto newLoads = [&](size_t g, std::vector<const View*>* out) -> size_t
        {
            size_t extra = 0;
            for (int k = 0; k < rj.numInputs; ++k)
            {
                const InputBinding& b = bindings[j][k];
                if (b.kind == InputBinding::ImmediateFill) continue;
                if (k == 1 && isRowReduction(rj.op)) continue;      // the destination is read by one thread per row, not as an operand
                if (b.kind == InputBinding::Producer && groupOf[b.producer] == g) continue;
                bool known = false;
                for (const View& v : groups[g].loads) if (v.sameElements(rj.in[k])) { known = true; break; }
                if (k == 1 && rj.in[1].sameElements(rj.in[0])) known = true;
                if (!known) { ++extra; if (out) out->push_back(&rj.in[k]); }
            }
            return extra;
        };
        size_t chosen = groups.size();
        if (limits.fusion)
        {
            for (size_t g = groups.size(); g-- > minGroup;)
            {
                if (groups[g].count != count || groups[g].ops.size() + 2 > limits.maxNodesPerKernel) continue;
                if (jReduces && groups[g].reductions + 1 > limits.maxReductionsPerKernel) continue;
                if (isRowReduction(rj.op) && groups[g].rowCols != 0 && groups[g].rowCols != rj.rowCols) continue;
                if (groups[g].loads.size() + groups[g].liveOutputs + newLoads(g, nullptr) + (liveOutput ? 1 : 0) > limits.maxTensorsPerKernel) continue;
                chosen = g;
                break;
            }
        }
        if (chosen == groups.size())
        {
            groups.emplace_back();
            groups.back().count = count;
        }
        std::vector<const View*> added;
        newLoads(chosen, &added);
        for (const View* v : added) groups[chosen].loads.push_back(*v);
        groups[chosen].liveOutputs += liveOutput ? 1 : 0;
        groups[chosen].reductions += jReduces ? 1 : 0;
        if (isRowReduction(rj.op)) groups[chosen].rowCols = rj.rowCols;
        groups[chosen].ops.push_back(j);
        groupOf[j] = chosen;
    }

    // ---- pass 2: which results must reach memory ---------------------------------------------------------------
    // A result is needed in memory when its storage is still alive after this batch, or when an op in another group
    // reads it.
    std::vector<char> readElsewhere(n, 0);
    for (size_t j = 0; j < n; ++j)
        for (int k = 0; k < ops[j].numInputs; ++k)
        {
            const InputBinding& b = bindings[j][k];
            if (b.kind == InputBinding::Producer && groupOf[b.producer] != groupOf[j]) readElsewhere[b.producer] = 1;
            if (b.kind == InputBinding::Memory)
            {
                // The reader goes to memory: every pending writer that overlaps the view must have stored by then.
                for (size_t i = 0; i < j; ++i)
                    if (meet(outRange[i], inRange[j][k]) && !superseded[i]) readElsewhere[i] = 1;
            }
        }

    // ---- pass 3: build one kernel per group --------------------------------------------------------------------
    std::vector<KernelSpec> kernels;
    kernels.reserve(groups.size());
    std::vector<int> nodeOf(n, -1);
    for (size_t g = 0; g < groups.size(); ++g)
    {
        const Group& grp = groups[g];
        KernelSpec spec;
        spec.count = grp.count;
        spec.opsFolded = static_cast<uint32_t>(grp.ops.size());

        auto findOrAddLoad = [&](const View& v) -> uint16_t
        {
            for (size_t l = 0; l < spec.loads.size(); ++l)
                if (spec.loads[l].view.sameElements(v)) return static_cast<uint16_t>(l);
            spec.loads.push_back({v, classifyAccess(v, grp.count)});
            return static_cast<uint16_t>(spec.loads.size() - 1);
        };
        auto addFillNode = [&](const OpRecord& fill) -> uint16_t
        {
            KernelNode node{};
            node.op = Op::Fill;
            node.dtype = fill.out.dtype;
            node.srcDtype = fill.out.dtype;
            node.scalarIndex = static_cast<uint16_t>(spec.scalars.size());
            spec.scalars.push_back(fill.scalar);
            spec.scalarDtypes.push_back(fill.out.dtype);
            spec.nodes.push_back(node);
            return static_cast<uint16_t>(spec.nodes.size() - 1);
        };

        for (size_t pos = 0; pos < grp.ops.size(); ++pos)
        {
            const size_t j = grp.ops[pos];
            const OpRecord& r = ops[j];
            OperandRef refs[2];
            for (int k = 0; k < r.numInputs; ++k)
            {
                const InputBinding& b = bindings[j][k];
                if (k == 1 && isRowReduction(r.op)) continue;       // the destination: handled with the reduction below
                if (b.kind == InputBinding::Producer && groupOf[b.producer] == g)
                {
                    refs[k].kind = OperandRef::Reg;
                    refs[k].index = static_cast<uint16_t>(nodeOf[b.producer]);
                }
                else if (b.kind == InputBinding::ImmediateFill)
                {
                    refs[k].kind = OperandRef::Reg;
                    refs[k].index = addFillNode(ops[b.producer]);
                    ++spec.fillsAbsorbed;
                }
                else
                {
                    refs[k].kind = OperandRef::Load;
                    refs[k].index = findOrAddLoad(r.in[k]);
                }
            }

            if (isReduction(r.op))
            {
                // the operand as a node: a register of this kernel, or an identity conversion of a loaded value
                uint16_t node = refs[0].index;
                if (refs[0].kind == OperandRef::Load)
                {
                    KernelNode copy{};
                    copy.op = Op::Cast;
                    copy.dtype = copy.srcDtype = r.in[0].dtype;
                    copy.a = refs[0];
                    spec.nodes.push_back(copy);
                    node = static_cast<uint16_t>(spec.nodes.size() - 1);
                }
                if (isRowReduction(r.op))
                {
                    KernelRowReduce rr{node, r.op == Op::MaxRows, r.in[0].dtype, r.out, false, 0};
                    if (bindings[j][1].kind == InputBinding::ImmediateFill)
                    {
                        const OpRecord& fill = ops[bindings[j][1].producer];
                        rr.initImmediate = true;
                        rr.scalarIndex = static_cast<uint16_t>(spec.scalars.size());
                        spec.scalars.push_back(fill.scalar);
                        spec.scalarDtypes.push_back(fill.out.dtype);
                        ++spec.fillsAbsorbed;
                    }
                    spec.rowReductions.push_back(rr);
                    spec.rowCols = r.rowCols;
                }
                else
                    spec.reductions.push_back({node, r.op == Op::MaxAll, r.in[0].dtype, r.out});
                continue;
            }
            if (r.op == Op::Fill)
            {
                nodeOf[j] = addFillNode(r);
            }
            else
            {
                KernelNode node{};
                node.op = r.op;
                node.dtype = r.out.dtype;
                node.srcDtype = r.numInputs > 0 ? r.in[0].dtype : r.out.dtype;
                node.a = refs[0];
                node.b = refs[1];
                spec.nodes.push_back(node);
                nodeOf[j] = static_cast<int>(spec.nodes.size() - 1);
            }

            // Is a later op of this group going to overwrite exactly the same elements?
            bool overwrittenLater = false;
            for (size_t later = pos + 1; later < grp.ops.size() && !overwrittenLater; ++later)
                overwrittenLater = ops[grp.ops[later]].out.sameElements(r.out);

            const bool alive = released.count(r.out.base) == 0;
            const bool store = readElsewhere[j] || (alive && !overwrittenLater && !superseded[j]);
            if (store)
            {
                // Replace an earlier store of this kernel to the same elements: only the last value must land.
                bool replaced = false;
                for (auto& st : spec.stores)
                    if (st.view.sameElements(r.out)) { st.node = static_cast<uint16_t>(nodeOf[j]); replaced = true; break; }
                if (!replaced)
                {
                    Access access = (r.out.isDense() || r.out.size == 1) ? Access::Dense : Access::General;
                    spec.stores.push_back({r.out, access, static_cast<uint16_t>(nodeOf[j])});
                }
            }
            else
            {
                ++spec.storesElided;
                if (r.op == Op::Fill) ++spec.fillsAbsorbed;
            }
        }
        if (!spec.stores.empty() || !spec.reductions.empty() || !spec.rowReductions.empty()) kernels.push_back(std::move(spec));
    }
    return kernels;
}

}   // namespace aixb200
