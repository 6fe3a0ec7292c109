# Times every example of this directory with the protocol of cuTile.jl's own benchmark driver (examples/benchmarks.jl
# there): 5 warm-up calls, 20 timed calls each between CUDA events, minimum and mean, throughput from each example's
# `metric`.  Usage: julia --project=.. benchmarks.jl [example names...].  Not executed in the build environment.
using CUDA, Printf

const NRUNS, WARMUP = 20, 5

rate(total, unit, ms) = unit == "GB/s" ? @sprintf("%.0f GB/s", total / ms / 1e6) :
                        unit == "TFLOPS" ? @sprintf("%.1f TFLOPS", total / ms / 1e9) : ""

function bench(name)
    m = Module(Symbol(name))
    Base.include(m, joinpath(@__DIR__, name * ".jl"))
    isdefined(m, :prepare) && isdefined(m, :run) || return
    data = Base.invokelatest(m.prepare; benchmark=true)
    res = Base.invokelatest(m.run, data; nruns=NRUNS, warmup=WARMUP)
    isdefined(m, :verify) && Base.invokelatest(m.verify, data, res)
    series = hasproperty(res, :times_fwd) ? Dict("cuTile Fwd" => res.times_fwd, "cuTile Bwd" => res.times_bwd) :
             res.times isa Dict ? res.times : Dict("B200" => res.times)
    met = isdefined(m, :metric) ? Base.invokelatest(m.metric, data) : nothing
    println("== ", name)
    for (label, ts) in sort(collect(series); by=first)
        total, unit = met isa Dict ? get(met, label, (0, "")) : met === nothing ? (0, "") : met
        @printf("  %-18s min %8.3f ms   mean %8.3f ms   %s\n", label, minimum(ts), sum(ts) / length(ts), rate(total, unit, minimum(ts)))
    end
end

names = isempty(ARGS) ? sort([replace(f, ".jl" => "") for f in readdir(@__DIR__) if endswith(f, ".jl") && f != "benchmarks.jl"]) : ARGS
foreach(bench, names)
