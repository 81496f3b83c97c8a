"""Codebooks of the GGUF IQ block formats (IQ2_XXS / IQ2_XS / IQ2_S, IQ3_XXS / IQ3_S, IQ1_S / IQ1_M).

A block of these formats stores indices into a fixed codebook of 4- or 8-value vectors; the codebooks are part of
the file format (ggml-common.h: iq2xxs_grid, iq2xs_grid, iq2s_grid, iq3xxs_grid, iq3s_grid, iq1s_grid).  Every entry
draws its values from a small alphabet, so an entry is kept here as one 16-bit number, the values' alphabet
positions as digits (first value = lowest digit), and a table as the base-85 text of its little-endian numbers.
:func:`grid` expands a table to a float tensor ``[entries, values per entry]``."""
import base64
import functools

import numpy as np
import torch

# name -> (values per entry, alphabet, entries, packed digits)
_TABLES = {
    "iq2xxs": (8, (8, 25, 43), 256,
        "000621ONsA2mlHI3;+@U6aW|i8UP#s9snc&DgZ73FaS0HH~>BXN&r#-Q~+84UI1(WiU5`Xq5z}-wgB1y^Z@n%`~U_42muZO5CIecAOR`?ECDhB"
        "J^@4lMgd9zRsm!Icma9=gaMoZo&m4{&H>;7<^k#f>;dut{s9641Of^I3<4qoIs#GxiUO1Z+5+4H;sWdf^a2J05(5|m90Mu?FataTP6Jj0U;~f?"
        "ngh%O(gWTD;sfpj0t74sOayKOd<4J*!UV_!+649l5Cs$kSOta!vIVpSx&_b$;05Rf>IEDIBnDIlRtBa9s0OYEzy{6+_68CMCI^NGo(HN2+6Pz&"
        "j0lbhln9y#o(P}_rU<MEv<SEe!U)6&$_U&D?g$DA5(yRwE(taXP6<{CU<rN+gb9!dv<bus+6m+dAPRB{bP9S3j0%tn!V2sP@Cy10G7C}*WD9Bw"
        "ZVPk^b_<#dpbNMQ(hC3#Mhun=m<+HC`V1fqN)1#ES`B&)whi(PKn_L@SPpOwjt;gC?hXtOFb^~jiVutrx(`4Q77-W`9uYDTP7!Jmb`gRR!VwA*"
        "3=$F&77`>9HWFGAdJ>!xvJ%D;*b@E{P!p&V@)P(I1QZGsI22A4b`-D_;uQ8202Npj3>G*R$`<Sv0v8|`Y8T2E(ij36"
    ),
    "iq2xs": (8, (8, 25, 43), 512,
        "000621ONsA2mlHI3;+%Q5C9SY6aW?g7yujq9snQ!A^;=+CIBb^DgZ73FaS0HH~=~TJODrdLI6epNB~j*Q~*{0SO8i8TmW7GU;ttOWB_IWYyfTm"
        "Z~$@ub^v$)egK33hyaQJkN~0pqyVM>r~s@0t^l+Ez5u`g#sJCy*Z|-F^Z@n%_yGC<`~dy{009C41_1~G4gnAW5&;we7y%jq904E!Dgi73G66&Z"
        "Mgd3xN&!v*Pyto}U;$zQXaRBodI6RJm;s&vtO2kAvH{Kk<^kvd>H+Kl?g8)t@&Wh(`~d<21Of^I5CR+mE&?_JI08BXKmt+%ZUS@yhyt1dpaRSS"
        "&;r^5+ydSL-~!?T<O1db=mP8l?gI1z_5%0<`U3s}00RaC4g(Ma5(5|mDg!J7E(0(FGy^sRJOf4pNCQp-U;}IeZUcM+egl95gaeiXr~}Lc&I8Z`"
        "(gW55*aO}J=mY8l?gQ`x`~w069t0o+CImPHZUlM+kOaU4!UV_!$^_a3<^=i#5Cs$kLIs8eum!ROv<0>WxCOceyam1m#0Aa;&;`~7=mq)(1O^5M"
        "3<e$sBnC7FR0e1UiUy(vrUs}6t_Hpazy|gP5(gXyJO@YzSO=5`m<OH*pa-f4zz5U^;s+cEC<s6ZObBuab_jR~j0lbhkO-0pln9mxm<XB(o(P}_"
        "rU<AAstBwIt_ZLQvIw{cya>Vw#0bg=+z8$X;0WRf<_PEr?g;n@`Un6C5(yRwCJ8PHFbOsZI0;4xNC|!kfC+*Lgb9cViV2PhkO`UzoC%@{v<bio"
        "&<WBB*a_qb>IoJKAPOi7J_<w%atd?`dJ2pRkP4UzpbEkY%nINN<_h)-77JtxW(#NwY71@)a0_+|d<%dJf(wWXnhUlIxC_1u!VAy~(hCL*Bn(yz"
        "SPWVWU<_&uatwqFjtrm-s0^+Q-VEdn3=J#|LJdj{Rt;tiZViwPtPQpexD6%_J`O+*Mh;jGWDaZ&cn*vXjt=w=0uLY$Fb_TtiVvI*pbyLsBoJ5-"
        "iV(^W>=5)277-W`8W9{3AQ2)FC=oCbG7&TpIuT3}P7!1gW)Wx+Y7uM^a1nwLj1iI%xDm<`?h)`201^fg3K9$w5)u>=77`>9HWEe>S`v5?rV_dm"
        ";1c{20uvGwC=)UhG!se_QWLTh)Dzkh;uGu>@DuVA_!9~g7!)WJKonFIa1^=}&J^Ml<`e)G1{DkyOcin!bQPc#`V}G;NEU<^q!!2)$`;NR&=%Sj"
        ";ua7WJ{Lq6W*2G~Y!`4BgcqO}vKQ7D{uhoIq8PRqz!<_9#u)Y({1^fmI2k$_Xc=l5kQtyE"
    ),
    "iq2s": (8, (8, 25, 43), 1024,
        "000621ONsA2mlHI3;+%Q5C9SY6aW?g7yujq9snQ!A^;=+CIBb^DgZ73FaR<DGypaLH~=~TJODrdLI6krOaM>-QUFu{RsdK4S^!)CUI1VKWB_IW"
        "YyfTmZ~$@ub^v$)dH{R?egJ|1gaC*DiU5!Rk^qzdngE;tq5z}-rU0k_tN^Y6v;e#Sz5u`g!T`ho#sJCy*Z|xB-~i+R>;Uut_5k<*`T+a@{r~_0"
        "0s#gA2muNK3;_-S5CIYa6af|i7y%jq9048yAORu)BmpV`ECDV7Faa_FHUT&RJOMrdL;*$tNC8R#OaV>-Pytc_Q~_22S^-=EU;$zQWC3OYXaQ;g"
        "YyoZoashM!dI5X^egS|1gaL*Di~*Jbm;ssroB^Hzq5-f0v;npOx&gca!U4<y&H>Z`<^kvd>H+Kl@B#7x^a1t(_yPO@00II61Of&E2m%TM3<3@U"
        "5CRke76KdsAOa`?HUc;TIs!lfLIOkrMgmF#QUX>2SOQ!EUIJtSZUS}!hys!VlmeUrpaP--tOCvg+5+4H-U8qP;sWFX<^t#f>;mor@B;J#_5%0<"
        "`U3s}00RO81Oo;G2m=ZO3<D4Y5(5+i7y}#w9s?o+Bm*h~ECVhBFat6JGy^sRI0HHZJOe%hKm$SpMgvF#N&`#-P6JQ_QUg>2SOZ!EU;|<UWCLac"
        "Y6ENod;@+1f&+vDhy#uTkOP(jnggH%q64x6v;(>W%mdB?&;!x~)&tlB+5_AJ-UH$T<OApf>I3Wp?gQ`x@&oh(_5=C@`~w061Ox^I2m}lS4g?eg"
        "9t0o+A_OD^CIl!1Dg-P9Fa$CLI0QNbJOn-jLIgwvN(58{Rs>uGZUk}!bOd+=dIW$3iUf=Vk_4m#z68Jo!UV(w#stU&%mmH^(gfNB+yveP-~{9Z"
        "<^=2n_5}C@5Cswi6a^Lq8U-8$A_Xi3E(J6NL<L#}WCdykd<BXHvIVpSwgtEayam1mzy-nu#0AI&%mvN`&;`~7*ag}J;sxjh@CEb*0tN&I1_lfU"
        "4h9eg76u*$AO<1^C<ZD9Fa|mXJO)ArR0doIXa;NsZU%A&cm|LLk_Ms%rUs}6ss^kEt_HFOv<A2ax(2`o!Un_!#s<m;%m&g1+y>qT<OcQz`Ud<4"
        "00#mG2nP}e6bBjyC<iPDNC!#>PzPcMatD|PoCl%@qzAMIwg<ci)(7YZ>Idux@&_ykLI_R>Y6x}+cnFLLjtGzlk_eOtmI#;#nh2Z-o(P}_q6nr4"
        "s0gYEtO%|Mun4jUv<S8cxCpukya>Vw#0bg=&Ir&5)CkrH+z8$X;0WRf<_PEr>Im!z?g;P*@(B0{`Uw08{s;gG0to~O1_=rY3<(km6bTjy7zrE+"
        "9tk7~E(tIRHVHThIte@pLJ3F-ObJd2QVCQES_xzcW(j@?fC+*Lgb9WThzW`bj0uhjkO`6rlnIsznhBf<o(Z4{q6wr4rU|GCtO>3Ov<bEexCy!m"
        "z6rny#tF~~(h1ZF)(O}N+6mkV-U;Ff<O%8t><R7(@Coz@_6ht61PTTU2nr4gAPOQ1Bnl=9DhezLG73BjJ_<w%Rtjtiatd?`cnW$7d<uRFfC_{P"
        "h6;=djtY<pk_wgzm<pZ>stT|Q!V1I+#tO&^%nHs5)C%4T;0opn_zDIK6blv$91AWBWD8~sXbWl!ZVPY=atm||b_;k5dJB9DfD3{PgbRiXhzp7f"
        "j0=tnk_(gznhTr@o(rH0qzk4CwhOomx(mDuz6-z$!VAO;$P3B~&<oNF)C<-N+6&wZ;tT8x?hEt_1`G-e3=9wq5)2p&A`B!9DhxUdJPcS2S`1ta"
        "UJPIiVhm&qW(;Z!Yz%S?bPRS3cno|Dehh>Rjtr0tmJFy2stl|Qt_-pav<$io#0<s^%naTP`V9OG0u2xi6b(uZObt#APz_WKRt;PYW({Z!ZVh$~"
        "fDN1to(-f8whinJ{0$}!Iu1S#Kn_9<Mh-|0N)Aj8P!3WKSPoncUJhaoWDaT$b`E?Fjt-Cxk`9y(m=2l_pbn}ItPZjc#17OB;tuEz`VI&WC=W0X"
        "G!HfpIuAS#LJv$2P7hQMW)Ff7gb#`joDZZAv=71$(hn36BoHPLED%%>Xb^M|ju7Gy4iOd+7!eu~91$Q9A`vDLC=o0XG7&TpIuSe(J`q3>L=j98"
        "P!U!USP^IuY7uS`a1nA5bP;wDdJ%jPf)Rufh7pJnj1i6zo)MrCrV+LgxDmV&z!Aa`#1YgH))Cwh3K9$w4iXR&5)u>=77`c|91<iFCK4zTDiSUd"
        "FcLNrKoUX{ND^8SToPUqU=m~!W)f@?b`p3JeiD!pm=dfKt`f8o#1h65{1N~Y1``Mq7!w*3AQMItP7_cQXcK-DvJ=P?$`jTT=o9c0@)PzG_!IgQ"
        "{1g5Y1QZGs3=|F&5EK*?78D#5CKM<XE)+l%L=;LCOcY!cUKC^$Y!s3dloXm2tQ6i9;uPc*<`n1@>=f=4^c4OS02Kxm7!@WJG!-@#JQYqAcolpV"
        "gcYO}v=!DB*cILt>=p18Bo-zXNES>Mwid`1%oflV)E3+p;uho<<`(Q05*HX3G#5%2Y!`ADeiwolgcqV0rWdFexEH(^z8Az7)))8}1{e$&92kNa"
        "wiw13_!uS`IvG|OSQ%m&WEp4~j2WOA"
    ),
    "iq3xxs": (4, (4, 12, 20, 28, 36, 44, 52, 62), 256,
        "000621ON#D3jhxQ5C9SY82};xI{-ZZK>$MlNB~LzQ2<o{SO8i8VE}9ZcmRL^f&hd7i2#rQk^q?in*g5xsQ|A4y#T=g#{kFx$^g{>_y7w59|0r*"
        "F9ACNJpn-hM*&&^Y5|=Av;oKg%mK~;;{ovj0RjU82m%TM5dsqe7y=ps90Df-C;~tNLIOzwPy$i{fdYd9hyscNkph?kx&pug!UE6&*#hPQ_5uL|"
        "1p_DpPy<v0W&?Qxg#*$9-~#{z0t5*J3j`1Z5(E|m83ZB(K?FktMFdC$N(4~^SOjwfcLaC@fCPdBi3E=XkOYzhp9G);tpvdY$OOy;_yqg}9R(`|"
        "Lj_j_VFi2z!3Dzw&IRQK0R{*L3I-7d69y;-H3m8cKn6kvPzG5BWCmsifd+#Hhz6Agss_3S$p+g77zZZ@ItM@pMh8*{Z3m18o(HoB+XwIm1PBiZ"
        "9S9!?D+n(Ld<c*Tp9r7`un4vY#|Y&J1PLh#GznD+V+nW(#R<p>$_dyB3JM_#I0`@tMhaF6Z3>JEnhLrK!V2pO2n!Pn7YjNILJL_7s0-8!;tLcE"
        "Bn&1DGz?J;aSV?Pv<%n`-V7uSMGa~Vn+?Ma(G3F*1r7%e2o4$!Dh^f-U=E57r4FhNzz)q0+Yay!5f32`Ko3F>R1cUB"
    ),
    "iq3s": (4, (1, 3, 5, 7, 9, 11, 13, 15), 512,
        "000310ssX72LK2F2>=QJ3;+%Q5C9PX6#yFmAOIo&B>*P?DF7<~FaR<DIRHEWKL9`gK>$JkL;y$tNdQd%PykZ^R{&W6T>xYNaR7AydH{d`fdGX7"
        "hX9BGivW%QkpPtdm;jsrq5!1;rvRw{s{ptFy8y!g$pFm&&;Zf^*#O%B-T>qP=m6>f_W=0-{Qv*~3jq%S5djnd8UY{yBLOJ^H~~TdL;+9%QUO*0"
        "TLEDKWdUaab^&_<h5?BIivgJdssXtHzyZPm!~xI&(gD^1+X3hS>;V7*0RjR71Of;G2?7fO4FV4W5CRec83G&v9s(=^E&?$EIs!lfK>|YpMgm9z"
        "Oaf5?SOQxDVFG9ZY65ryegc33iUN%Sj{=YalmeOppaP=;tpczDx&pxh!~(|x$O6j((E`^3*aF-F;R5mk_yPk11p^8L3<DVh8v`N(CIct~ECWFU"
        "NCQg)Q3F^5S_5eVkOPzhmjk2&rUStP!vn|z$^+2@-2>qR@&ot-00aR90|W&G2LuQN3Iq%U4g?Vd69g9o7z7#wAp|1?B?Kr0Dg-wKI0QQcJp@1m"
        "LIg+zO9W2@QUp~5Sp-}JVgzXffdqsEhXj!XlLVLqp9G-<s|2qExdglfzy!hs#RSO&(gf55*#z4J;sodf_5=Y12L%uX69pOt9R(o;It4uiL<LC&"
        "QUzZHU<GRhcm;q3f(3^Kkp-;<u?58i$pzL0*ahPS=mi1>2?h%W4F(Se5(XIt8wMQ)A_gP|Ck817GX^;ZK?XwxMFva;Q3g{6U<PmodIo+5fCh>N"
        "kOrCtoCc@{!3M|%%m&d0(+1ZD*aqPS;|Avj?FRb>0|yBQ4hIqk83!r{Fb6aTK?g_&N(WU3S_fnYZU=h@jt8L!!3V<!&<D~7-3I^&1PBTU5C{|q"
        "7YG^%AqXf4I0!-rM+iv>O9)a3SO{GRV+d&oZ3uw~g9wNSjR=tln+Tu?uL!aTxCq1u$q35`&<N59*$CYT00{yK6bT;*APG4MMF~d<Q3-MhiwT?w"
        "unEWs%?a2E;|b{r0tyHU3<?qoAPOW3CkiSGHVQlnK?*|(MG8s^Q3_fLdJ2FFi3*bnm<pZ>s|vyj#|p>_*9znc=?e7<`w9UI1Pc%g8Ve>1N()vC"
        "X$xx$q6@+c#0%032@DGi4Gb9!8w@ZEKnzd}R}6FviVU0#q71DJvJAKkzzoa`(G1`W6%8W|G7UftLk(OFa1DhGpbg0l%MAby1P%ud5DpR!9u6Q5"
        "EDkabLJmm|R1RYfWe$N3gbs)fjt-Fym=389!VcOF-45#x0S^Ta3l9(vC=XH(Vh@53nGe7Z"
    ),
    "iq1s": (8, (-1, 0, 1), 2048,
        "000621ONsA2mlHI4FD1V6aW|i8UP;vB>*P?DF875HUKyPJODlbLjXtsN&rp(Pykc_RRCK6T>xJIVE|$PX8>&gaR74wcK~?+eE@#|fdGR5gaC^G"
        "kpPnbl>nUpq5z}-r~s+}uK=_Fwg9>Sya2%f#{kU$(g4-~*Z|r9-T>eL;sE6U=m6>f>;Uip@&Nq+{{R622>}lQ6#*Lo9|0o)Bmpx4IRQTbMFB?v"
        "NC8O!Q2|o{RRLWAUjbtQX8~vdX#r~iYyoWnZvk-ua{+Y$cL8|;djW(2hXIKJivf)Rj{%SYkpYtdp#h}<u>rFIxdFQYy#c=g!U4kp#{tO!&jHl|"
        "*8$rB<^kvd>;dip^8xq)`T_m{00IR93jz-U7Xlmt9s(i)BmyY{E&?zDGy*mPI|4xhLjp$vOae^;QvzE8TmoMLWddgcYXWxyc>;R^eFB35hyscN"
        "jslPZl>(XqoC2T%q5`J^tpc+GwgR~Vz5>7k!UDts#sbR%&;rr|)&kf9;sWCW<pSvf?gH-u^#b<-{Q?040|N&G2?GiP4Feei8v`8!A_FA@D+4V9"
        "F9R_HGXpgPHv>5XJp(@jLjy?zO#@B?PXkZ`Q3Fx~Qv+24R|8uEV*_ggZ3A-ybpwS1hXaWNkpq?kn**H#p#!4>r30q}s{^eAwFA2Yy#v1k#{<m+"
        "(F4;1*aO)E+XLJK-vi?V=mYBm>;vrs?*s7z^8@q)^#k_<`vd(0{{saC2?PrS4g?Pb5d;zh69g3m7X%mt8w4K&Ap|7^Cj==3Dg-M8Ed(zFF$6ON"
        "H3T;VIRrZdJOn)iLIgtuL<B_yMg&L%Nd!v-O$1H^PXti}Qv_86Rs>fBSp-`ITm)SNUj$$TVFY6YWCUddX9Q^kZv=4!as+b(djxz0eFT35fdqvF"
        "i3E!Tj0BAYj|7nflLVFomjsvunFO2!o&=u+p#-7?qXel0tOTzFu>`pUy#&bw%>>m1+XUSN-vr?V;{@jf=>+Qp>;&xu?*#D#^91<>{{#UA3k4Yk"
        "8wDK&Aq67^CIu}8E(I?IF$FaRHw8EaIR!ffJOw=kK?OwxO$AT|Q3X>4RRviET?JnSXa#Qtb_I9^e+7XBg9U{JhXsiRiv^DblLeIpn+2f-r3I)3"
        "vIVpSxCOcezXikv#s$a)$_2~?(FNB9-38zU;|1si>ILov@CEe+`UU(2{sjOA0tN>L4F(Se69yRuAO;}@B?c=7Ee0<JF$OaRGzK*WJqAJsM+Qj-"
        "PX<*6S_WJOUIt+XW(H^mYzA%ya|U?^eFlF9g$9cTkOq<llm?duoCcl-q6VY}sRpqIvj(*Wy9UDs#0JF%#|Fy=%?8f~(FWHB-v;Fd=LYKr?gsG&"
        "{RRUE2?q}c5eF3q7Y7>$9S0r<AqOP~CkH79GY2&XI0rcgI|n@nKL<evLkC3%O9xN~QU_NDT?b<aX$NlybO&_@dk26Af(M2Njt7_rng^Z-pa-P~"
        "st2qGum`dSw+FokzX!<&&Iiy3)CblF;0NLd<_G8p@CWk;^#}O}{|5;O3kVMg5eOFu83-E)9S9=`C<rYGF9<XUH3&KgJP1GtLI_L<P6$#6R0vrJ"
        "UkGCeWe95sa0qe;b_jR~eF%aGgb0WTiU^Mgl?a&#p$M%Au?VvWwFtKexd^)my$H<+(FoKC*a+MR-3Z?Z;Rxdh=LqQt>Imxy?FjD(^9c0_`w0CA"
        "{|EsI0|^8P1qlZU2nh`d4+#+o6A2Xw7YQ2)9SI)^Bnc%6CJ8YKHwifjI|)MxNeNR4RS8)MT?t_cY6))%c?o|BiwTYimkFH-p9!G}qY0%6rU|DB"
        "tO>0NuL-dUvkA2cxe2=oy$Qbw!3o9*#|g~|&<W8A(+SrJ*$LYT+zH(Y-wELf<q7Et>j~`%?g{S+@d@(@^a=I}_X+q3`3d?7{R#gG015#L0}2NU"
        "2nq=b3knYk5egCt6ABdy777~*9SR=`Aqpf4CkiYIEebCRF$yyZH3~TjI|@AtKMFw#L<&U;MhZv@NeW8}PYO{AQwmoKS_)nYVhUplX$or!Z3=Y?"
        "dkTIEf(nNUjtY|sl?s^(n+l%_p$el4r3$MGu?n*awF<Wiy$Zt$#tO#@$_mR0&I->8(F)ZH*9zGR-3s9f<qGEt=nCly>I&-$?F#P-@e1<_^a}S1"
        "{R;mI0}BNU1`7uZ3kwYk4+{|sAqz1JGYd5fI}1GvKMO+(M+;R8UkhamXA5WxX$xx$Zwqk?bqjY3c?*3De+z>Pg$s!biwlekjSG(pl?#^(p9`T2"
        "rwgeItP8CRu?w>cxeL1sybHYxzYD<&!VAL-#0$j>#|z5~%nQv6&kNBD(+kuK)eF}P*$dhW+Y8(a-3#6e-wWUi;S1vn<qPHu=L_iz?F;V<^$Yh4"
        "_zU?9`wRUG0SpBU2Mh}g5eyRy7YrE;8w?{1B@8JHD-10RE(|XWF$^^fHw-`wMGQv_NeoO3O$<>CS`1qZVGLsoWDI2tW(;QxY7A`*Zwzq^a}0G1"
        "b_{n6c?^0CdklOGehhyMfDC~Qf((NUg$#xahYW}ei42PjjSQ0vl?;~*nGBi?n+%-{pbVl6qYS4EsSK(Ns|>6RtqiXWu?(^dvkbHhwG6flxD2@r"
        "y9~Vyz6`$%!3@I;#0<p@#tg>{$PCF0$_&g5%?!>A&kWEE(G1cI(+t!M)eP1Q*bLbW+6>za+zj0e-wfdl;tb^s<_zZy=nU!%>kRA+?F{Y=@eK0}"
        "^bGY3_YC<A`V9LF{0#mK{|o>P0}TZY1`P-e2@MMk3=Itp4h;_t5DgIx5)Bm%7!4T>8Vwr_91R@}9t|H2APpf6A`K%ABn>4ECk-hLDh(|SF%2^f"
        "Gz~QkHVrooISo7wKn+6;MGZy`M-4~~O$|;BPYqEGQw>)QSq)tcWDRKzYYlA;Zw+w`at(70bPaV4cMW+BdJTIGf(?fai4BVljSY_tlMR^-oDH1~"
        "pADl8r46SIs12zNs|~RYw+*=sx(&Mxy$!z&zzx9-!VSX>#0|v_#tp{}$qma5%ni*A&kfQI)eYDU+YQ|f-VNUk;0@so=MC=-@(uY7{SE#N0uBQX"
        "1r7@i4Gs<t5e^g%6%G~-7Y-W^9S$E3Ar2!BDh@3UFAgvcF%B~hH4Z@zNe)X6O%78ITMl6kWe#QzXAWr&YYuG=Zw_$|bPj<Ii4Knrkq(m%l@6H>"
        "n+~B4q7J1Frw*+Sunw~hwhp%rxemV$zz)L>#}3R6&koTJ*ACkb-45vv?GEn_`VRXJ{|*Na2oDJl3=bI(9}goBD-SvkI}be%J`X_;Lk~v}Ne@d8"
        "O%G2GQ4doORS#DWSPxkbTMt|hT@POmVGn5!Y7cD>Zx3+~au0J4bPsh8cMo|Fdk=pPg%5`hi4Thpjt`Fykq@5_pbw!BqYtGIrVpqOsSm0TtPigb"
        "u@ABjvk$coybrz)zYoC=#1F*}#}CL4%MZ;D&JWKI)DPJY-w)&u=@04;>ksV@@elJ4^$+(C`49RJ`w#pN{ty2T0}ure2oMSo3=j|y6c82=7Z4Z_"
        "8W0^29}prCF%UBlIS@Y(Nf1jAPY_WMR}ftgV-RQ%a1eD6cMyFLfe?ofi4cnrjS!CzkPwp)ln|8=nGl;0oDiK5pAexCr4XqQtPrgbvJkfry%4_;"
        "z!1X_&k)lP)DYni;}GW%=@9J@?-212^$_+D`49jR2N4Pp3=t9$77-W`91$K7C=n_VE)g&hH4!=yI}tq*KM_F@M-faBP7zWOR1sMbUJ+msWD#Z&"
        "YY}k~a}jkBcM*LNgAs)hi4lttjS-I#kP(p)k`b2?nGu^2p%J7JsS&FYtr4>kxDmP$z7fC?#SzL8%n{HL(h=Pe-x1>x=@IS`@DcP8_7VFL01^Tc"
        "1`-Go6%rW|B@!nRE)p>kH4--xITAe*OA=2KTM}UsWfEr+YZ7r1a}sqDb`p6KdlG*Vff9legA#=jh7yYsj1r9!j}nm*lM<B@mlBy0n-ZN8pAx4M"
        "wGz1!yAr_?#}dgB%@WQM&l1xT))Lne*%I9n;1cB$>k{%3_7eOO{t^Nc1QQ7p4igX)6cZK`7!w;4Arm7LClf6bFcUHpG!r-zIukz=L=#36N)t>I"
        "Q4>-VR})ziTN7gwX%lM`Z4+-3aT9YBbrX3LdlP*VhZB(#lM|T}o)e%Gq!XqSs}ryjvJ<uwxD&k-!xP05#}m{O))U$j+!Nsw<`d`>>=W)2^Aq_K"
        "{S*EZ{}Tli3lt9&5fm2`85A27BNQYQDHJahF%&ZtH55A(K@>w2MHELANfb>KPZUuUQxsJcR}@(kTNGauWE5o-XB21@X%uS|ZxnG9c@%pTffR!j"
        "g%pVtixiC%j}(;@n-rZCp%kYSuN1KqvlO)yw-mV)yA;C|#T3gF(-hSd;1uH&<rL=>>lE)4@f7(K{S*Zi2Nekw3Ka_#3>6I(4;2s<5fu{^8x<WD"
        "BNZeSB^4(XD-|&nGZi-#ITbq<JQY0^KNUa~K@~$4MiogFOchNPPZd!WQWaAbRTWniSQS|nS`}LrToqjvUKL*zVHIN)WEEu<XBBD{Z53}7a}{(I"
        "brp6McNKXRdKG&WeHDKdffa)lg%yVtjTMm<logg0n-!fEqZOqUrWL6bsuipitrf2owH3D&ycN9_!4<+4#TCXC#}&^N(G}Ab*%jjz<rV7{@fGzI"
        "`4#&W{T2Qd0Tu-o1{Mz%6&4v58x|oJDHbahEfy~pF%~lxH5NA(I2Jh;I~F|_K^8+6MHWXENft{MO%_fTPZm)YRTftkSQc9rT^3&!Wfo@^X%=l3"
        "Zx(YFdlrNijTV&_mll~8n--rIp%$eUu@<)$xfZ$>yB5e6$`;NR&=%De+7{dv;1=Q*=N9c2?-ubE^A`RV02c%o1{Vt#5El{`78e*79Ty-MBNrtX"
        "Cl@IfDi=8yI~P6|K^H?8MHfdGNf%QWSQlCsT^C;$Y!`4Bau;(KdKZ2df)|7ri5HI-lNXg2n-`!Lq8FwYs28mlvKO=$xEHz?%NNlX*B99r-xuN+"
        ";}_)@=NIW0>=*49?icSD^%oHs6Brd37Z@2B8yF)PB^W6fD;O~tGZ-`&H5fM-Js3e4Ll{LEMi@sJNf=ESPZ&`cVHjr^YZz`Aa2RtKdl-EffEa@q"
        "g&2kyhZu?&j2M_0oEV@Op%|kWrWmLgsu->quo$!$wiv(|!WhOF$QaWY)fm?p*%;&)<{0W2>=^MF_89mW{22Zi0~re$4;c~}6&V{DBN-<dD;X^r"
        "F&Q%%J{dz9P#IDgRvB0sVi{x^Xc=l5bs2XVc^QToh#8C-jv12~m>HTGo*AGS"
    ),
}


@functools.lru_cache(maxsize=None)
def grid(name: str) -> torch.Tensor:
    """Codebook ``name`` (``iq2xxs``, ``iq2xs``, ``iq2s``, ``iq3xxs``, ``iq3s``, ``iq1s``) as float32 ``[entries, 4 or 8]``."""
    width, alphabet, entries, text = _TABLES[name]
    codes = np.frombuffer(base64.b85decode(text), dtype="<u2").astype(np.int64)
    assert codes.size == entries
    base = len(alphabet)
    digits = (codes[:, None] // base ** np.arange(width)[None, :]) % base
    return torch.from_numpy(np.asarray(alphabet, dtype=np.float32)[digits])


def signs7() -> torch.Tensor:
    """[128, 8] of +1 / -1: a 7-bit sign field gives the signs of seven values, the eighth makes the number of
    negative ones even (ggml-common.h: ksigns_iq2xs)."""
    i = torch.arange(128)
    bits = (i.unsqueeze(1) >> torch.arange(8)) & 1
    bits[:, 7] = bits[:, :7].sum(1) & 1
    return 1.0 - 2.0 * bits.float()
